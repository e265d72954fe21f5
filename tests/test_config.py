import json
import glob
import os

import pytest

from open_transformers_b200.config import compose, load_config, parse_config_resolved
from open_transformers_b200.config.load import default_configs_dir
from open_transformers_b200.train.checkpoint import resolved_config_json


def test_every_train_recipe_loads():
    names = [os.path.basename(p)[:-5] for p in glob.glob(str(default_configs_dir() / "train" / "*.yaml"))]
    assert {"100m_smoke_repop", "1b_repop_v2", "1b_midtrain_math", "open1b_b200", "tiny_cpu"} <= set(names)
    for n in names:
        cfg = load_config(n)
        assert cfg.data.seq_len == cfg.train.seq_len


def test_open1b_shape_and_window_rule():
    cfg = load_config("1b_repop_v2")
    m = cfg.model
    assert (m.n_layers, m.d_model, m.n_heads, m.n_kv_heads, m.head_dim, m.ffn_intermediate, m.vocab_size) == (24, 2048, 16, 4, 128, 5632, 128256)
    assert cfg.train.total_tokens == 400_000_000_000 and cfg.train.global_batch_tokens.late == 9_437_184
    full = [i for i in range(24) if m.layer_window(i) == 0]
    assert full == [4, 9, 14, 19, 23]
    assert m.qk_norm_gain is False and cfg.train.spike.grad_norm_threshold == 5.0


def test_overrides_and_group_choice():
    cfg = load_config("tiny_cpu", ["train.grad_clip=0.5", "++run.tp_size=2", "optim.peak_lr=1e-4", "schedule=wsd"])
    assert cfg.train.grad_clip == 0.5 and cfg.run.tp_size == 2 and cfg.optim.peak_lr == 1e-4 and cfg.schedule.name == "wsd"
    with pytest.raises(KeyError):
        compose("tiny_cpu", ["train.no_such_key=1"])
    with pytest.raises(KeyError):
        compose("tiny_cpu", ["+train.grad_clip=1"])


def test_unknown_key_and_validators():
    with pytest.raises(Exception):
        load_config("tiny_cpu", ["++model.typo=1"])
    with pytest.raises(Exception):
        load_config("tiny_cpu", ["model.vocab_size=1000"])
    with pytest.raises(Exception):
        load_config("tiny_cpu", ["model.swa_window=48"])
    with pytest.raises(Exception):
        load_config("tiny_cpu", ["data.seq_len=256"])
    with pytest.raises(Exception):  # halt can never trigger: 4 * 5 > 10
        load_config("tiny_cpu", ["train.spike.halt_window_steps=10"])
    for bad in (["model.d_model=130"], ["model.n_kv_heads=3"], ["++model.qat.weight_bits=9"], ["++model.qat.act_bits=1"], ["optim.peak_lr=-1"],
                ["optim.betas=[1.2,0.9]"], ["optim.eps=0"], ["train.micro_batch_size=0"], ["schedule.min_lr_frac=1.5"], ["train.grad_clip=-1"],
                ["model.z_loss.coeff=-1"], ["train.state_hash.every_n_steps=-1"]):
        with pytest.raises(Exception):
            load_config("tiny_cpu", bad)
    assert load_config("tiny_cpu", ["train.grad_clip=0", "++model.qat.weight_bits=4"]).model.qat.weight_bits == 4


def test_resolved_config_round_trip_and_retired_keys():
    cfg = load_config("100m_smoke_repop")
    blob = resolved_config_json(cfg)
    assert parse_config_resolved(blob) == cfg
    import json

    d = json.loads(blob)
    d["train"]["clip_algo"] = "per_tensor"  # a key an older checkpoint may carry
    assert parse_config_resolved(d) == cfg


def test_describe_lists_every_schema_leaf_and_prints_resolved_recipes(capsys):
    import yaml

    from open_transformers_b200.config.describe import main, schema_rows

    rows = {k: (kind, default) for k, kind, default in schema_rows()}
    assert rows["run.tp_size"] == ("int", "1") and rows["model.n_layers"][1] == "(required)" and rows["train.spike.start_step"][0] == "int"
    cfg = load_config("tiny_cpu")

    def leaves(d, prefix=""):
        for k, v in d.items():
            if isinstance(v, dict):
                yield from leaves(v, prefix + k + ".")
            else:
                yield prefix + k

    resolved = set(leaves(json.loads(cfg.model_dump_json())))
    listed = set(rows)
    # every scalar of a resolved recipe is a listed key (lists of sources / names are listed as one key)
    assert {k for k in resolved if not k.startswith("data.sources")} <= listed | {"optim.betas"}, sorted(resolved - listed)[:5]
    assert main([]) == 0 and "train.grad_clip" in capsys.readouterr().out
    assert main(["--config-name", "tiny_cpu", "train.grad_clip=0.25"]) == 0
    assert yaml.safe_load(capsys.readouterr().out)["train"]["grad_clip"] == 0.25
