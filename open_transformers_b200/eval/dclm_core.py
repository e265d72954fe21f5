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


# --------------------------------------------------------------------------------------------------------------------
# The runner behind ``pretrain-eval``: the loglikelihood slice of DCLM-CORE that is scored per checkpoint, grouped into
# categories; each task goes through the lm-eval harness with the model wrapped by ``eval/lm_eval_adapter.PretrainLM``.
# Generative tasks are left out (no KV cache: they would dominate the cost). The result file is what
# ``scripts/plot_evals.py`` reads. (task grouping, few-shot counts and the JSON layout: reference
# src/pretrain/eval/dclm_core.py:33-129)
CORE_CATEGORIES: dict[str, list[str]] = {
    "commonsense": ["hellaswag", "piqa", "winogrande"],
    "world_knowledge": ["mmlu"],
    "reading": ["boolq", "openbookqa"],
}
CORE_FEWSHOT: dict[str, int] = {"mmlu": 5}   # every other task is zero-shot
_PRIMARY_KEYS = ("acc_norm,none", "acc,none", "exact_match,none", "pass_at_1,none")


def primary_metric(metrics: dict) -> float:
    """The score a task is tracked by: normalised accuracy where the harness reports it, else accuracy, exact match,
    pass@1, else the first number in the dict, else 0."""
    for key in _PRIMARY_KEYS:
        if key in metrics:
            return float(metrics[key])
    for value in metrics.values():
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
    return 0.0


def _harness_evaluate(model, tokenizer, device):
    """``evaluate(task, num_fewshot) -> metrics`` over lm-eval; raises when the harness is not installed."""
    from lm_eval import evaluator

    from .lm_eval_adapter import PretrainLM

    lm = PretrainLM(model, tokenizer, device=device)

    def evaluate(task: str, num_fewshot: int) -> dict:
        return evaluator.simple_evaluate(model=lm, tasks=[task], num_fewshot=num_fewshot).get("results", {}).get(task, {})

    return evaluate


def run_dclm_core(model, tokenizer, out_dir, step: int, task_subset: dict[str, list[str]] | None = None, device="cuda", evaluate=None) -> dict:
    """Score the registered tasks and write ``<out_dir>/step_<step, 9 digits>.json``:
    {"step", "tasks": {name: {"primary", "all"} | {"error"}}, "categories": {category: mean of its tasks' primaries},
    "category_tasks", "macro_average": mean over categories}. Without the harness the file holds {"step", "error",
    "categories": {}}. ``evaluate(task, num_fewshot) -> metrics`` replaces the harness (tests, other scorers)."""
    import json
    import logging
    from pathlib import Path

    log = logging.getLogger(__name__)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    target = out / ("step_%09d.json" % step)
    if evaluate is None:
        try:
            evaluate = _harness_evaluate(model, tokenizer, device)
        except Exception as e:  # the harness is an optional dependency
            log.warning("lm-eval unavailable (%s); writing an empty result", e)
            result = {"step": step, "error": str(e), "categories": {}}
            target.write_text(json.dumps(result, indent=2))
            return result
    groups = task_subset or CORE_CATEGORIES
    tasks, categories = {}, {}
    for category, names in groups.items():
        scores = []
        for name in names:
            try:
                metrics = evaluate(name, CORE_FEWSHOT.get(name, 0))
                tasks[name] = {"primary": primary_metric(metrics), "all": metrics}
                scores.append(tasks[name]["primary"])
            except Exception as e:
                log.warning("task %s failed: %s", name, e)
                tasks[name] = {"error": str(e)}
        if scores:
            categories[category] = sum(scores) / len(scores)
    result = {"step": step, "tasks": tasks, "categories": categories, "category_tasks": {c: list(n) for c, n in groups.items()},
              "macro_average": sum(categories.values()) / len(categories) if categories else 0.0}
    target.write_text(json.dumps(result, indent=2))
    log.info("DCLM CORE @ step %d: macro=%.4f categories=%s", step, result["macro_average"], {k: round(v, 4) for k, v in categories.items()})
    return result
