"""OLMES evaluation of a checkpoint, two ways.

* With AllenAI's ``oe_eval`` (the OLMES reference implementation) and ``lm_eval`` installed, `run_olmes` drives
  ``oe_eval.run_eval.run_eval`` as a library: suite names are expanded to leaf task configs (`expand_olmes_tasks`, what
  the olmes launcher does before it calls ``run_eval``), the decoder is handed over as an ``HFLM_Verbose`` whose "HF model"
  is `HFStyleModel` (lm-eval only touches ``.device``, ``.config``, ``.tie_weights()`` and ``forward().logits``), and
  ``metrics-all.jsonl`` is distilled into ``summary.json`` by `summarize_metrics` (aggregates, the 10-task macro, extended
  tasks). Generation tasks decode greedily row by row without a KV cache: the decoder takes no attention mask, so a
  left-padded batch would attend to its padding (reference src/pretrain/eval/olmes_runner.py:172-398).
* Without them (this image has neither, and no network), `run_task_files` scores multiple-choice JSONL task files with
  the same wrapper: every choice of a question in one forward pass, per-token and summed log-likelihood normalisations.

Inputs are right-padded to a multiple of 32 positions; the causal mask keeps padding from reaching a real position
(reference :134-151).
"""
from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

PAD_MULTIPLE = 32
OLMES_DEFAULT_SUITES = ["core_9mcqa::olmes", "mmlu::olmes"]
OLMES_EXTENDED_TASKS = ["agi_eval_english:1shot::olmes", "mmlu_pro:mc::none", "naturalqs::olmes", "drop::olmes", "triviaqa::olmes",
                        "gsm8k::olmes"]
OLMES_MAX_LENGTH = 2048
EOS_TOKEN, BOS_TOKEN, PAD_TOKEN = "<|endoftext|>", "<|begin_of_text|>", "<|pad|>"


@dataclass
class CausalLMOutput:
    logits: torch.Tensor


class HFStyleModel(torch.nn.Module):
    """What lm-eval's HFLM needs of a ``transformers`` model, around the decoder."""

    def __init__(self, model, tokenizer=None, device=None, pad_id: int | None = None):
        super().__init__()
        self.model, self.tokenizer = model.eval(), tokenizer
        self._device = torch.device(device) if device is not None else next(model.parameters()).device
        self.pad_id = pad_id if pad_id is not None else (tokenizer.eos_id if tokenizer is not None else 0)
        self.config = type("Cfg", (), {"model_type": "open_transformers_b200_llama3", "vocab_size": model.cfg.vocab_size,
                                       "max_position_embeddings": model.cfg.max_seq_len_pretrain})()

    @property
    def device(self) -> torch.device:
        return self._device

    def tie_weights(self) -> None:  # HFLM calls it on every model; the head here is untied
        return None

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask=None, **_) -> CausalLMOutput:
        B, T = input_ids.shape
        pad = (-T) % PAD_MULTIPLE
        if pad:
            input_ids = torch.cat([input_ids, input_ids.new_full((B, pad), self.pad_id)], 1)
        out = self.model(input_ids.to(self._device))
        logits = out.logits if hasattr(out, "logits") else out
        return CausalLMOutput(logits[:, :T].float())

    def to(self, *_a, **_k):
        return self


@torch.no_grad()
def score_multiple_choice(hf_model: HFStyleModel, context: str, choices: list[str], normalise: str = "per_token") -> dict:
    tok = hf_model.tokenizer
    ctx = tok.encode(context) or [tok.eos_id]
    conts = [tok.encode(ch) for ch in choices]
    # all choices of a question in ONE forward pass: rows right-padded to the longest
    width = max(len(ctx) + len(c) for c in conts)
    ids = torch.tensor([ctx + c + [tok.eos_id] * (width - len(ctx) - len(c)) for c in conts])
    logits = hf_model(ids).logits
    scores = []
    for i, cont in enumerate(conts):
        lp = torch.log_softmax(logits[i, len(ctx) - 1: len(ctx) + len(cont) - 1].float(), -1)
        s = float(lp.gather(-1, torch.tensor(cont, device=lp.device)[:, None]).sum()) if cont else 0.0
        scores.append(s / max(len(cont), 1) if normalise == "per_token" else s)
    return {"scores": scores, "prediction": max(range(len(choices)), key=scores.__getitem__)}


def run_task_files(hf_model: HFStyleModel, task_files: list[str], limit: int | None = None) -> dict:
    """{task name: {"accuracy" (per-token normalisation), "accuracy_raw" (summed), "n"}} over JSONL files of
    {"context", "choices", "answer"} rows; the task is named after its file."""
    tasks = {}
    for tf in task_files:
        rows = [json.loads(line) for line in Path(tf).read_text().splitlines() if line.strip()][:limit]
        hit = {"per_token": 0, "sum": 0}
        for r in rows:
            for norm in hit:
                hit[norm] += score_multiple_choice(hf_model, r["context"], r["choices"], norm)["prediction"] == r["answer"]
        n = max(len(rows), 1)
        tasks[Path(tf).stem] = {"accuracy": hit["per_token"] / n, "accuracy_raw": hit["sum"] / n, "n": len(rows)}
    return tasks


# ------------------------------------------------------------------------------------------ oe_eval integration
def olmes_available() -> bool:
    import importlib.util

    return all(importlib.util.find_spec(m) is not None for m in ("oe_eval", "lm_eval"))


def build_hf_tokenizer(tokenizer_path: str | Path):
    """The run's ``tokenizer.json`` as a ``transformers`` fast tokenizer with the special tokens registered (the file is
    in HF ``tokenizers`` format already; a registered pad token keeps lm-eval from re-purposing eos)."""
    from transformers import PreTrainedTokenizerFast

    return PreTrainedTokenizerFast(tokenizer_file=str(tokenizer_path), eos_token=EOS_TOKEN, bos_token=BOS_TOKEN, pad_token=PAD_TOKEN)


def greedy_generate(call_model, context: torch.Tensor, attention_mask: torch.Tensor, stop: list[str] | None, max_new: int, eot_id: int,
                    pad_id: int, decode) -> dict:
    """Greedy decoding in the shape of HF ``generate`` output: {"sequences": [B, ctx + gen] (rows padded with ``pad_id``
    after their end), "scores": one [B, vocab] tensor per generated position}. Each row is decoded on its own from its
    un-padded prefix, one full forward per token."""
    B, ctx_len = context.shape
    produced_rows, score_rows = [], []
    for b in range(B):
        prefix = context[b][attention_mask[b].bool()].tolist()
        produced, scores = [], []
        for _ in range(max(int(max_new), 1)):
            logits = call_model(torch.tensor([prefix + produced], dtype=torch.long, device=context.device))[0, -1].clone()
            scores.append(logits)
            nxt = int(logits.argmax())
            produced.append(nxt)
            if nxt == eot_id or (stop and any(s in decode(produced) for s in stop)):
                break
        produced_rows.append(produced)
        score_rows.append(scores)
    gen = max(len(p) for p in produced_rows)
    sequences = torch.full((B, ctx_len + gen), pad_id, dtype=torch.long, device=context.device)
    sequences[:, :ctx_len] = context
    out_scores = torch.zeros((B, gen, score_rows[0][0].shape[-1]), device=context.device)
    for b, (produced, scores) in enumerate(zip(produced_rows, score_rows)):
        sequences[b, ctx_len:ctx_len + len(produced)] = torch.tensor(produced, dtype=torch.long, device=context.device)
        out_scores[b, :len(scores)] = torch.stack(scores)
    return {"sequences": sequences, "scores": tuple(out_scores[:, t] for t in range(gen))}


def build_lm(model, hf_tokenizer, device, batch_size: int, max_length: int):
    """The olmes LM adapter (an ``HFLM_Verbose``) around a ready-made decoder."""
    from lm_eval.models.huggingface import HFLM
    from oe_eval.models.eleuther_huggingface import HFLM_Verbose

    class OlmesLM(HFLM_Verbose):
        def __init__(self):
            HFLM.__init__(self, pretrained=HFStyleModel(model, None, device, pad_id=0), tokenizer=hf_tokenizer, backend="causal",
                          batch_size=int(batch_size), max_length=int(max_length))
            self.tokenizer_size = len(self.tokenizer)

        def _model_generate(self, context, attention_mask, stop, **kw):
            if kw.get("do_sample") or (kw.get("temperature") or 0.0) > 0.0:
                raise NotImplementedError("greedy decoding only")
            max_new = int(kw.get("max_length", context.shape[1] + self.max_gen_toks)) - context.shape[1]
            return greedy_generate(self._model_call, context, attention_mask, stop, max_new, self.eot_token_id, self.tokenizer.pad_token_id,
                                   self.tok_decode)

    return OlmesLM()


def expand_olmes_tasks(specs: list[str], suites: dict | None = None, task_configs: dict | None = None) -> list[dict]:
    """Suite and task names -> leaf task configs (deep copies), each tagged with ``metadata.alias`` = its name, which
    the suite aggregation in ``oe_eval`` matches on. ``suites`` / ``task_configs`` default to oe_eval's tables."""
    if suites is None or task_configs is None:
        from oe_eval.configs.task_suites import TASK_SUITE_CONFIGS
        from oe_eval.configs.tasks import TASK_CONFIGS

        suites = TASK_SUITE_CONFIGS if suites is None else suites
        task_configs = TASK_CONFIGS if task_configs is None else task_configs
    leaves: list[str] = []
    todo = list(reversed(specs))
    seen_suites: set[str] = set()
    while todo:
        name = todo.pop()
        if name in suites:
            if name in seen_suites:
                raise ValueError("suite %r contains itself" % name)
            seen_suites.add(name)
            todo.extend(reversed(suites[name]["tasks"]))
        else:
            leaves.append(name)
    out = []
    for name in leaves:
        if name not in task_configs:
            raise ValueError("unknown olmes task %r" % name)
        cfg = copy.deepcopy(task_configs[name])
        cfg.setdefault("metadata", {})["alias"] = name
        out.append(cfg)
    return out


def run_olmes(model, tokenizer_path: str | Path, out_dir: str | Path, tasks: list[str] | None = None, extended: bool = False,
              batch_size: int = 4, max_length: int = OLMES_MAX_LENGTH, limit: int | None = None, device="cuda",
              model_label: str = "open_transformers_b200") -> dict:
    """Run OLMES suites through ``oe_eval`` on a ready-made decoder. Per-task output lands in ``out_dir``
    (``metrics-all.jsonl``, predictions); the returned summary is also written to ``summary.json`` there. ``limit`` caps
    the instances per task: smoke runs only, the scores stop being comparable."""
    import oe_eval.run_eval as oe_run

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    specs = list(tasks or OLMES_DEFAULT_SUITES)
    if extended:
        specs += [t for t in OLMES_EXTENDED_TASKS if t not in specs]
    configs = expand_olmes_tasks(specs)
    if limit is not None:
        for cfg in configs:
            cfg["limit"] = limit
    argv = ["--task", *[json.dumps(c) for c in configs], "--model", model_label, "--model-type", "hf", "--output-dir", str(out_dir),
            "--batch-size", str(batch_size), "--max-length", str(max_length)]
    args = vars(oe_run._parser.parse_args(argv))
    lm = build_lm(model, build_hf_tokenizer(tokenizer_path), device, batch_size, max_length)
    stock_loader = oe_run.load_model  # oe_eval has no registry for model back-ends: its loader is swapped for the run
    oe_run.load_model = lambda _cfg: lm
    try:
        oe_run.run_eval(args)
    finally:
        oe_run.load_model = stock_loader
    return summarize_metrics(out_dir)


def summarize_metrics(out_dir: str | Path) -> dict[str, Any]:
    """``metrics-all.jsonl`` -> ``summary.json``: ``aggregates`` (rows without a task index: per-task best-of-MC/RC and
    the suite macros), the count of core-suite formulation leaves, ``extended_tasks`` and ``olmes_macro`` = the 10-task
    headline (nine core tasks and MMLU, one vote each)."""
    out_dir = Path(out_dir)
    aggregates, leaves, extended = {}, {}, {}
    for line in (out_dir / "metrics-all.jsonl").read_text().splitlines():
        if not line.strip():
            continue
        row = json.loads(line)
        score = (row.get("metrics") or {}).get("primary_score")
        if score is None:
            continue
        alias = ((row.get("task_config") or {}).get("metadata") or {}).get("alias", row.get("task_name"))
        if row.get("task_idx") is None:
            aggregates[alias] = score
        elif alias.endswith("::olmes") and (":mc::" in alias or ":rc::" in alias):
            leaves[alias] = score
        else:
            extended[alias] = score
    core, mmlu = aggregates.get("core_9mcqa::olmes"), aggregates.get("mmlu::olmes")
    summary: dict[str, Any] = {"olmes_macro": None if core is None or mmlu is None else (9 * core + mmlu) / 10,
                               "aggregates": aggregates, "num_leaf_tasks": len(leaves)}
    if extended:
        summary["extended_tasks"] = extended
    (out_dir / "summary.json").write_text(json.dumps(summary, indent=2))
    return summary
