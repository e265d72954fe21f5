"""Evaluation stack on the CPU against a tiny trained checkpoint: sliding-window perplexity, the lm-eval style
adapter, the HF-style wrapper with the multiple-choice scorer, the ``pretrain-eval-olmes`` CLI with its run-directory
summary, and the plot script that reads those summaries."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import tiny_cfg
from open_transformers_b200.cli.eval import load_model_from_checkpoint
from open_transformers_b200.cli.eval_olmes import main as olmes_main
from open_transformers_b200.data.tokenizer import Tokenizer, train_tokenizer
from open_transformers_b200.eval.lm_eval_adapter import PretrainLM
from open_transformers_b200.eval.olmes_runner import HFStyleModel, score_multiple_choice
from open_transformers_b200.eval.perplexity import perplexity, sliding_window_nll
from open_transformers_b200.train.loop import train

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("evalrun")
    cfg = tiny_cfg(str(tmp), ["train.ckpt_every_steps=3", "model.vocab_size=512"])
    res = train(cfg, device="cpu", data_root=str(tmp))
    step_dir = sorted((Path(res["run_dir"]) / "checkpoints").glob("step_*"))[-1]
    texts = ["the quick brown fox jumps over the lazy dog %d times" % i for i in range(200)]
    tok_path = train_tokenizer(iter(texts), tmp / "tok.json", vocab_size=300, min_frequency=1)
    return str(step_dir), str(tok_path), res["run_dir"]


def test_perplexity_windows_cover_every_token_once(ckpt):
    model, cfg, _ = load_model_from_checkpoint(ckpt[0], "cpu")
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, 512, (200,), generator=g)
    nll_a, n_a = sliding_window_nll(model, tokens, 64, 64)
    nll_b, n_b = sliding_window_nll(model, tokens, 64, 32)   # overlapping windows score each token once as well
    assert n_a == n_b == 199
    assert nll_a > 0 and nll_b > 0
    for stride in (64, 32):   # several windows per forward pass: same sum
        nll_1, n_1 = sliding_window_nll(model, tokens, 64, stride)
        nll_4, n_4 = sliding_window_nll(model, tokens, 64, stride, batch_windows=4)
        assert n_1 == n_4 == 199 and abs(nll_1 - nll_4) <= 1e-6 * nll_1
    ppl = perplexity(model, tokens, 64)
    assert math.isfinite(ppl) and 50 < ppl < 5000            # an untrained 512-way model sits near the vocabulary size


def test_adapter_and_multiple_choice(ckpt):
    model, _, _ = load_model_from_checkpoint(ckpt[0], "cpu")
    tok = Tokenizer(ckpt[1])
    lm = PretrainLM(model, tok, max_length=64)
    (lp, greedy), = lm.loglikelihood([("the quick brown", " fox")])
    assert lp < 0 and isinstance(greedy, bool)
    (roll,) = lm.loglikelihood_rolling(["the lazy dog jumps"])
    assert roll < lp
    (text,) = lm.generate_until([("the quick", ["\n"])], max_new_tokens=4)
    assert isinstance(text, str)
    hf = HFStyleModel(model, tok)
    out = hf(torch.tensor([tok.encode("the quick brown fox")]))
    assert out.logits.shape[-1] == 512 and out.logits.shape[1] == len(tok.encode("the quick brown fox"))
    r = score_multiple_choice(hf, "the quick brown", [" fox", " dog", " cat"])
    assert len(r["scores"]) == 3 and r["prediction"] in (0, 1, 2)


def test_batched_scoring_equals_one_request_at_a_time(ckpt):
    model, _, _ = load_model_from_checkpoint(ckpt[0], "cpu")
    tok = Tokenizer(ckpt[1])
    reqs = [("the quick brown", " fox"), ("", " the lazy dog jumps over"), ("the quick brown fox jumps over the lazy dog 17 times and", " again"),
            ("dog", " times 3"), ("the lazy", " dog 12 times"), ("over the", " lazy")]
    one = PretrainLM(model, tok, max_length=64).loglikelihood(reqs)
    many = PretrainLM(model, tok, max_length=64, batch_size=4).loglikelihood(reqs)
    assert [g for _, g in one] == [g for _, g in many]
    assert all(abs(a - b) <= 1e-5 * max(1.0, abs(a)) for (a, _), (b, _) in zip(one, many)), (one, many)
    texts = ["the lazy dog jumps", "the quick brown fox jumps over the lazy dog " * 12]      # the second spans several windows
    r1 = PretrainLM(model, tok, max_length=64).loglikelihood_rolling(texts)
    r4 = PretrainLM(model, tok, max_length=64, batch_size=4).loglikelihood_rolling(texts)
    assert all(abs(a - b) <= 1e-5 * abs(a) for a, b in zip(r1, r4)) and r1[1] < r1[0]


def test_olmes_cli_writes_the_summary_the_plot_script_reads(ckpt, tmp_path, capsys):
    task = tmp_path / "toy_task.jsonl"
    task.write_text("\n".join(json.dumps({"context": "the quick brown", "choices": [" fox", " dog"], "answer": i % 2}) for i in range(4)))
    assert olmes_main(["--checkpoint", ckpt[0], "--tokenizer", ckpt[1], "--task-file", str(task), "--run-dir", ckpt[2]]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert set(line["tasks"]) == {"toy_task"} and line["tasks"]["toy_task"]["n"] == 4
    summaries = list((Path(ckpt[2]) / "evals_olmes").glob("step_*/summary.json"))
    assert len(summaries) == 1 and json.loads(summaries[0].read_text())["macro"] == line["macro"]
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "plot_evals_olmes.py"), ckpt[2], "-o", str(tmp_path / "o.png")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert (tmp_path / "o.png").exists() or "macro" in r.stdout


def test_lockstep_generation_equals_one_request_at_a_time(ckpt):
    model, _, _ = load_model_from_checkpoint(ckpt[0], "cpu")
    tok = Tokenizer(ckpt[1])
    reqs = [("the quick", ["\n"]), ("the lazy dog jumps over the quick brown", None), ("fox", ["zzz"]), ("", None), ("dog 17 times", [" "])]
    one = PretrainLM(model, tok, max_length=64).generate_until(reqs, max_new_tokens=6)
    many = PretrainLM(model, tok, max_length=64, batch_size=3).generate_until(reqs, max_new_tokens=6)
    assert one == many and len(one) == 5


def test_multiple_choice_scores_in_one_pass_equal_one_choice_at_a_time(ckpt):
    model, _, _ = load_model_from_checkpoint(ckpt[0], "cpu")
    tok = Tokenizer(ckpt[1])
    hf = HFStyleModel(model, tok)
    ctx, choices = "the quick brown", [" fox", " dog jumps over the lazy", " cat 7"]
    got = score_multiple_choice(hf, ctx, choices, normalise="sum")["scores"]
    c = tok.encode(ctx)
    for ch, g in zip(choices, got):
        k = tok.encode(ch)
        lp = torch.log_softmax(hf(torch.tensor([c + k])).logits[0, len(c) - 1: -1].float(), -1)
        want = float(lp.gather(-1, torch.tensor(k)[:, None]).sum())
        assert abs(want - g) <= 1e-5 * max(1.0, abs(want))


def test_eval_command_scripts_and_core_aggregate(ckpt, tmp_path, capsys):
    """pretrain-eval on a held-out shard with a task-accuracy file; the DCLM-CORE style aggregate; the curve-plotting,
    system-information and prompt scripts as a user runs them"""
    import numpy as np

    from open_transformers_b200.cli.eval import main as eval_main
    from open_transformers_b200.data.indexed_dataset import IndexedDatasetWriter
    from open_transformers_b200.eval.dclm_core import DCLM_CORE_TASKS, centred, dclm_core_score

    rng = np.random.default_rng(0)
    with IndexedDatasetWriter(tmp_path / "heldout", np.uint32) as w:
        for _ in range(6):
            w.add_document(rng.integers(0, 512, 90).astype(np.uint32))
    acc = {"arc_easy": 0.40, "piqa": 0.60, "lambada_openai": 0.10, "not_a_core_task": 0.99}
    (tmp_path / "acc.json").write_text(json.dumps(acc))
    capsys.readouterr()
    assert eval_main(["--checkpoint", ckpt[0], "--held-out", str(tmp_path / "heldout"), "--max-tokens", "300", "--batch-windows", "2", "--no-dclm",
                      "--out-dir", str(tmp_path / "ev"), "--task-accuracies", str(tmp_path / "acc.json")]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out == json.loads((tmp_path / "ev" / "summary.json").read_text())
    assert out["held_out_tokens"] == 300 and 50 < out["held_out_ppl"] < 5000 and "dclm_core_macro" not in out
    want = {"arc_easy": (0.40 - 0.25) / 0.75, "piqa": (0.60 - 0.5) / 0.5, "lambada_openai": 0.10}
    assert out["dclm_core"]["per_task"] == pytest.approx(want) and out["dclm_core"]["core"] == pytest.approx(sum(want.values()) / 3)
    assert "not_a_core_task" not in out["dclm_core"]["per_task"] and len(out["dclm_core"]["missing"]) == len(DCLM_CORE_TASKS) - 3
    assert centred(1.0, 0.25) == 1.0 and centred(0.25, 0.25) == 0.0 and dclm_core_score({})["core"] == 0.0
    # the DCLM-CORE slice: without the harness an empty result file and the reason; with a scorer handed in, the categories,
    # the single-task category, a failing task, and the file scripts/plot_evals.py reads
    from open_transformers_b200.eval.dclm_core import primary_metric, run_dclm_core

    with pytest.raises(SystemExit):
        eval_main(["--checkpoint", ckpt[0]])                                   # the task run needs a tokenizer
    assert eval_main(["--checkpoint", ckpt[0], "--tokenizer", ckpt[1], "--out-dir", str(tmp_path / "ev2")]) == 0
    out2 = json.loads(capsys.readouterr().out)
    empty = json.loads(next((tmp_path / "ev2").glob("step_*.json")).read_text())
    if "dclm_core_error" in out2:                                              # lm-eval is not installed here
        assert empty["categories"] == {} and empty["error"] == out2["dclm_core_error"] and out2["dclm_core_macro"] is None
    scores = {"hellaswag": {"acc_norm,none": 0.30, "acc,none": 0.28}, "piqa": {"acc,none": 0.60}, "mmlu": {"acc,none": 0.27}, "boolq": {"exact_match,none": 0.5}}
    shots = {}

    def scorer(task, num_fewshot):
        shots[task] = num_fewshot
        return scores[task]                                                   # winogrande and openbookqa raise KeyError: recorded as errors

    run_dir = Path(ckpt[2])
    for step, bump in ((10, 0.0), (20, 0.05)):
        scores["piqa"] = {"acc,none": 0.60 + bump}
        res = run_dclm_core(None, None, run_dir / "evals" / ("step_%d" % step), step, evaluate=scorer)
    assert shots["mmlu"] == 5 and shots["piqa"] == 0 and "error" in res["tasks"]["winogrande"] and res["tasks"]["hellaswag"]["primary"] == 0.30
    assert res["categories"] == pytest.approx({"commonsense": (0.30 + 0.65) / 2, "world_knowledge": 0.27, "reading": 0.5})
    assert res["macro_average"] == pytest.approx(sum(res["categories"].values()) / 3) and res["category_tasks"]["world_knowledge"] == ["mmlu"]
    assert (run_dir / "evals" / "step_20" / "step_000000020.json").exists() and primary_metric({"note": "x", "f1": 0.4}) == 0.4 and primary_metric({}) == 0.0
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "plot_evals.py"), str(run_dir), str(run_dir), "--stitch", "-o", str(tmp_path / "e.png")],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert (tmp_path / "e.png").exists() or ("mmlu" in r.stdout.splitlines()[0] and r.stdout.count("\n") >= 3)
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "plot_training_curves.py"), str(run_dir / "logs" / "metrics.jsonl"), "--out", str(tmp_path / "c.png")],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert (tmp_path / "c.png").exists() or r.stdout.count("\n") >= 3          # a figure, or the CSV dump where matplotlib is absent
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "collect_system_info.py")], capture_output=True, text=True, timeout=300)
    info = json.loads(r.stdout)
    assert r.returncode == 0 and info["cpu"]["logical_cpus"] >= 1 and "version" in info["torch"] and isinstance(info["env"], dict)
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "prompt_checkpoint.py"), "--checkpoint", ckpt[0], "--tokenizer", ckpt[1], "--prompt", "the quick",
                        "--max-new-tokens", "3", "--temperature", "0"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.startswith("the quick"), r.stderr[-2000:]


def test_olmes_suites_through_a_stand_in_for_oe_eval(ckpt, tmp_path, monkeypatch):
    """`run_olmes` against stand-ins for the two packages it drives (neither is installed here): suite names expand to
    leaf configs tagged with their alias, every leaf travels as one JSON argument, the library's model loader is swapped
    for ours during the run and put back after, and metrics-all.jsonl is distilled into summary.json."""
    import json
    import sys
    import types

    from open_transformers_b200.eval import olmes_runner as R

    suites = {"core_9mcqa::olmes": {"tasks": ["arc_easy::olmes", "pair"]}, "pair": {"tasks": ["boolq:mc::olmes", "boolq:rc::olmes"]},
              "mmlu::olmes": {"tasks": ["mmlu_x:mc::olmes"]}}
    configs = {n: {"task_name": n.split(":")[0], "num_shots": 5} for n in ("arc_easy::olmes", "boolq:mc::olmes", "boolq:rc::olmes",
                                                                            "mmlu_x:mc::olmes", "gsm8k::olmes")}
    leaves = R.expand_olmes_tasks(["core_9mcqa::olmes", "gsm8k::olmes"], suites, configs)
    assert [c["metadata"]["alias"] for c in leaves] == ["arc_easy::olmes", "boolq:mc::olmes", "boolq:rc::olmes", "gsm8k::olmes"]
    assert "metadata" not in configs["arc_easy::olmes"]                       # the tables themselves are not edited
    with pytest.raises(ValueError):
        R.expand_olmes_tasks(["no_such_task"], suites, configs)
    with pytest.raises(ValueError):
        R.expand_olmes_tasks(["loop"], {"loop": {"tasks": ["loop"]}}, configs)

    seen = {}

    class FakeHFLM:
        max_gen_toks = 4

        def __init__(self, pretrained=None, tokenizer=None, backend=None, batch_size=1, max_length=0):
            self.model, self.tokenizer, self.batch_size, self.max_length = pretrained, tokenizer, batch_size, max_length

        def _model_call(self, ids):
            return self.model(ids).logits

        def tok_decode(self, ids):
            return " ".join(map(str, ids))

        eot_token_id = 0

    import argparse

    parser = argparse.ArgumentParser()
    parser.add_argument("--task", nargs="+")
    for flag in ("--model", "--model-type", "--output-dir", "--batch-size", "--max-length"):
        parser.add_argument(flag)

    def fake_run_eval(args):
        lm = oe_run.load_model({})
        seen["lm"], seen["args"] = lm, args
        ids = torch.randint(1, 200, (2, 5))
        out = lm._model_generate(ids, torch.ones_like(ids), stop=None, max_length=8)
        seen["generated"] = out["sequences"].shape, len(out["scores"])
        rows = [{"task_name": "core_9mcqa", "task_idx": None, "task_config": {"metadata": {"alias": "core_9mcqa::olmes"}}, "metrics": {"primary_score": 0.5}},
                {"task_name": "mmlu", "task_idx": None, "task_config": {"metadata": {"alias": "mmlu::olmes"}}, "metrics": {"primary_score": 0.3}},
                {"task_name": "boolq", "task_idx": 1, "task_config": {"metadata": {"alias": "boolq:mc::olmes"}}, "metrics": {"primary_score": 0.6}},
                {"task_name": "gsm8k", "task_idx": 3, "task_config": {"metadata": {"alias": "gsm8k::olmes"}}, "metrics": {"primary_score": 0.1}},
                {"task_name": "broken", "task_idx": 4, "metrics": {}}]
        (Path(args["output_dir"]) / "metrics-all.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")

    oe_run = types.ModuleType("oe_eval.run_eval")
    oe_run._parser, oe_run.run_eval, oe_run.load_model = parser, fake_run_eval, "the stock loader"
    mods = {"oe_eval": types.ModuleType("oe_eval"), "oe_eval.run_eval": oe_run, "oe_eval.configs": types.ModuleType("oe_eval.configs"),
            "oe_eval.configs.task_suites": types.ModuleType("oe_eval.configs.task_suites"),
            "oe_eval.configs.tasks": types.ModuleType("oe_eval.configs.tasks"), "oe_eval.models": types.ModuleType("oe_eval.models"),
            "oe_eval.models.eleuther_huggingface": types.ModuleType("oe_eval.models.eleuther_huggingface"),
            "lm_eval": types.ModuleType("lm_eval"), "lm_eval.models": types.ModuleType("lm_eval.models"),
            "lm_eval.models.huggingface": types.ModuleType("lm_eval.models.huggingface")}
    mods["oe_eval"].run_eval = oe_run
    mods["oe_eval.configs.task_suites"].TASK_SUITE_CONFIGS = suites
    mods["oe_eval.configs.tasks"].TASK_CONFIGS = configs
    mods["lm_eval.models.huggingface"].HFLM = FakeHFLM
    mods["oe_eval.models.eleuther_huggingface"].HFLM_Verbose = type("HFLM_Verbose", (FakeHFLM,), {})
    for name, mod in mods.items():
        monkeypatch.setitem(sys.modules, name, mod)
    monkeypatch.setattr(R, "build_hf_tokenizer", lambda path: type("Tok", (), {"pad_token_id": 3, "__len__": lambda self: 256})())

    model, _cfg, _eng = load_model_from_checkpoint(ckpt[0], "cpu")
    summary = R.run_olmes(model, ckpt[1], tmp_path / "olmes", tasks=["core_9mcqa::olmes", "mmlu::olmes"], extended=False, batch_size=2,
                          max_length=64, limit=7, device="cpu", model_label="m")
    assert oe_run.load_model == "the stock loader"                            # put back after the run
    sent = [json.loads(t) for t in seen["args"]["task"]]
    assert [t["metadata"]["alias"] for t in sent] == ["arc_easy::olmes", "boolq:mc::olmes", "boolq:rc::olmes", "mmlu_x:mc::olmes"]
    assert all(t["limit"] == 7 for t in sent) and seen["args"]["batch_size"] == "2" and seen["args"]["model_type"] == "hf"
    assert seen["generated"][0][0] == 2 and 1 <= seen["generated"][1] <= 3 and seen["generated"][0][1] == 5 + seen["generated"][1]
    assert summary["olmes_macro"] == pytest.approx((9 * 0.5 + 0.3) / 10) and summary["num_leaf_tasks"] == 1
    assert summary["extended_tasks"] == {"gsm8k::olmes": 0.1} and summary["aggregates"]["mmlu::olmes"] == 0.3
    assert json.loads((tmp_path / "olmes" / "summary.json").read_text()) == summary


def test_olmes_cli_says_what_is_missing_without_oe_eval(ckpt, capsys):
    assert olmes_main(["--checkpoint", ckpt[0], "--tokenizer", ckpt[1], "--out-dir", "/tmp/never_written"]) == 2
    assert "oe_eval" in capsys.readouterr().err


def test_system_snapshot_sections_fake_gpu_inventory_and_redaction(tmp_path, monkeypatch):
    """Every section is there, a broken probe costs only its own section, the GPU inventory comes from nvidia-smi's query
    output (a stand-in executable here, which only answers reads), and variables that look like secrets are redacted."""
    import importlib.util
    import stat

    spec = importlib.util.spec_from_file_location("collect_system_info", ROOT / "scripts" / "collect_system_info.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fake = tmp_path / "nvidia-smi"
    row = "0, NVIDIA B200, GPU-abc, 580.159, 97.00, 183359, 12, 1965, 1965, 3996, 3996, 180.5, 1000.00, 41, Enabled, Default, Enabled, Disabled, 5, 16"
    fake.write_text("#!/bin/sh\ncase \"$*\" in *query-gpu*) echo '%s'; echo '%s' | sed 's/^0/1/';; *topo*) echo 'GPU0 GPU1 NV18';; *) echo links;; esac\n" % (row, row))
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + ":" + __import__("os").environ["PATH"])
    monkeypatch.setenv("WANDB_API_KEY", "do-not-print")
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    monkeypatch.setenv("UNRELATED_SETTING", "x")
    monkeypatch.setitem(mod.PROBES, "memory", lambda: 1 / 0)
    info = mod.collect([ROOT])
    for section in ("host", "kubernetes", "cpu", "memory", "disk", "network", "gpu", "nvidia_driver", "cuda", "python", "torch", "kernels", "git", "env", "pip_freeze"):
        assert section in info, section
    assert info["memory"] == {"error": "ZeroDivisionError: division by zero"} and info["cpu"]["logical_cpus"] >= 1
    assert info["gpu"]["count"] == 2 and info["gpu"]["devices"][1]["name"] == "NVIDIA B200" and info["gpu"]["devices"][0]["clocks.max.sm"] == "1965"
    assert "NV18" in info["gpu"]["topology"]
    assert info["env"]["WANDB_API_KEY"] == "<redacted>" and info["env"]["NCCL_NVLS_ENABLE"] == "0" and "UNRELATED_SETTING" not in info["env"]
    assert set(info["kernels"]["native_source_digests"]) >= {"otb_cpu"} and str(ROOT) in info["git"]
    assert "2 x NVIDIA B200 driver=580.159" in mod.summary_line(info)
    out = tmp_path / "deep" / "pod-0.json"
    assert mod.main(["--output", str(out)]) == 0 and json.loads(out.read_text())["schema_version"] == 1


def test_prompt_session_commands_change_the_sampler_and_reject_nonsense(ckpt):
    import importlib.util
    import io

    spec = importlib.util.spec_from_file_location("prompt_checkpoint", ROOT / "scripts" / "prompt_checkpoint.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["prompt_checkpoint"] = mod                                     # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    out = io.StringIO()
    sess = mod.Session(mod.Settings(), out)
    assert not sess.command("once upon a time")
    for line in (":temp 0", ":topk 5", ":topp 0.5", ":tokens 3", ":seed 7", ":show"):
        assert sess.command(line)
    assert (sess.s.temperature, sess.s.top_k, sess.s.top_p, sess.s.max_new_tokens, sess.s.seed) == (0.0, 5, 0.5, 3, 7)
    for line in (":temp hot", ":topp 1.5", ":tokens 0", ":tokens", ":frobnicate 1"):
        assert sess.command(line)
    assert (sess.s.temperature, sess.s.top_p, sess.s.max_new_tokens) == (0.0, 0.5, 3)          # nothing changed
    text = out.getvalue()
    assert "not a number: hot" in text and "top_p out of range" in text and ":tokens needs a value" in text and "unknown command :frobnicate" in text
    assert "temperature=0 top_k=5 top_p=0.5 max_new_tokens=3 seed=7" in text
    with pytest.raises(SystemExit):
        sess.command(":quit")
    model, cfg, _ = load_model_from_checkpoint(ckpt[0], "cpu")
    tok = Tokenizer(ckpt[1])
    out.seek(0)
    out.truncate()
    a = sess.complete(model, tok, "the quick", "cpu", cfg.train.seq_len)
    assert a.startswith("the quick") and out.getvalue().rstrip("\n") == a            # what was streamed is what was returned
    sess.command(":seed 7")
    assert sess.complete(model, tok, "the quick", "cpu", cfg.train.seq_len, stream=False) == a   # greedy: the same text again
