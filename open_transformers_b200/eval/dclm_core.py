"""DCLM-CORE style aggregate: a fixed task list with random-guess baselines; the score is the macro average
of centred accuracies (acc - baseline) / (1 - baseline) (reference src/pretrain/eval/dclm_core.py)."""
from __future__ import annotations

DCLM_CORE_TASKS: dict[str, float] = {
    "arc_easy": 0.25, "arc_challenge": 0.25, "hellaswag": 0.25, "piqa": 0.5, "winogrande": 0.5, "boolq": 0.5, "copa": 0.5,
    "openbookqa": 0.25, "commonsense_qa": 0.2, "lambada_openai": 0.0, "squad": 0.0, "coqa": 0.0, "bigbench_qa_wikidata": 0.0,
    "jeopardy": 0.0, "agi_eval_lsat_ar": 0.25, "bigbench_dyck_languages": 0.0, "bigbench_operators": 0.0,
    "bigbench_repeat_copy_logic": 0.0, "bigbench_cs_algorithms": 0.0, "bigbench_language_identification": 0.25,
    "winograd": 0.5, "mmlu_fewshot": 0.25,
}


def centred(acc: float, baseline: float) -> float:
    return (acc - baseline) / (1.0 - baseline) if baseline < 1.0 else 0.0


def dclm_core_score(accuracies: dict[str, float]) -> dict:
    used = {t: centred(a, DCLM_CORE_TASKS[t]) for t, a in accuracies.items() if t in DCLM_CORE_TASKS}
    missing = sorted(set(DCLM_CORE_TASKS) - set(used))
    return {"core": sum(used.values()) / max(len(used), 1), "per_task": used, "missing": missing}
