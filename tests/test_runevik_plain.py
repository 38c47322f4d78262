"""Runevik without a GPU: the configuration parser, the tensor list, random model folders, and the plain
implementation against itself (a prompt at once against the same tokens one by one)."""
import copy

import pytest
import torch

import tiny_runevik as tr
from helpers import load_plain, random_tokens
from plain_runevik import PlainRunevik, short_conv, sinusoid


def test_config_becomes_parts_and_schedule():
    from nanoinfer_b200.config import config_from_dict
    cfg = config_from_dict(tr.R1)
    assert cfg.architecture == "Runevik" and cfg.hidden_size == 96 and cfg.vocab_size == 300
    assert [l.mixer.kind for l in cfg.layers] == ["latent_attention", "gated_delta", "latent_attention", "gated_delta"]
    assert [r.cache_of for r in cfg.schedule] == [None, None, 0, None]
    assert cfg.layers[3].feed_forward is None and cfg.layers[0].feed_forward.intermediate_size == 160
    assert cfg.layers[1].mixer.extra_dict() == {"value_dim": 40, "conv_taps": 3, "norm_eps": 1e-5}
    assert cfg.layers[2].mixer.softmax_scale == 0.2 and cfg.layers[2].mixer.extra_dict()["own_latent"] is False
    assert all(l.arrangement == "parallel" and l.mixer_norm.kind == "rmsnorm_scalar" for l in cfg.layers)
    assert cfg.embedding.kind == "table_sinusoid" and cfg.embedding.extra_dict()["layer_inputs"] == 4 * 8
    assert "layer_inputs" not in config_from_dict(tr.R2).embedding.extra_dict()


def test_tensor_names_and_shapes():
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.plan import tensor_plan
    plan = {p.name: p.shape for p in tensor_plan(config_from_dict(tr.R1))}
    assert plan["embed"] == (300, 96) and plan["side.embed"] == (300, 32) and plan["head"] == (300, 96)
    assert plan["final.norm"] == () and plan["l0.norm1"] == ()
    assert plan["l0.mix.dkv"] == (48, 96) and plan["l0.mix.dkv.norm"] == (48,) and plan["l0.mix.uk"] == (48, 48)
    assert plan["l0.mix.uv"] == (72, 48) and plan["l0.mix.g"] == (3, 96)
    assert "l2.mix.dkv" not in plan and "l2.mix.dkv.norm" not in plan and plan["l2.mix.uk"] == (64, 48)
    assert plan["l1.mix.q"] == (24, 96) and plan["l1.mix.k.conv"] == (24, 3) and plan["l1.mix.v"] == (80, 96)
    assert plan["l1.mix.v.conv"] == (80, 3) and plan["l1.mix.A_log"] == (2,) and plan["l1.mix.norm"] == (40,)
    assert plan["l1.mix.g"] == (80, 96) and plan["l1.mix.o"] == (96, 80) and plan["l1.mix.b"] == (2, 96)
    assert plan["l1.mlp.up"] == (136, 96) and plan["l1.mlp.act"] == (4,) and "l3.mlp.up" not in plan
    assert plan["l3.side.gate"] == (8, 96) and plan["l3.side.proj"] == (96, 8) and plan["l3.side.norm"] == (96,)
    assert not any(n.startswith("l0.side") for n in tensor_plan_names(tr.R2))


def tensor_plan_names(raw):
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.plan import tensor_plan
    return [p.name for p in tensor_plan(config_from_dict(raw))]


@pytest.mark.parametrize("change, message", [
    (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=1), "latent of its own"),
    (lambda r: r["layers"][2]["mixer"].update(kv_rank=32), "differ in kv_rank"),
    (lambda r: r["layers"][1].update(type="window"), "not a mixer"),
    (lambda r: r["layers"][1]["mixer"].update(heads=3, kv_heads=2), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mlp"].update(kind="routed"), "not supported"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_bad_configs_are_refused(change, message):
    from nanoinfer_b200.config import ConfigError, config_from_dict
    raw = copy.deepcopy(tr.R1)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_random_model_folder_loads(tmp_path):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.weights import load_weights
    tr.write_model(str(tmp_path / "m"), tr.R3, seed=3)
    cfg = load_config(str(tmp_path / "m"))
    w = load_weights(str(tmp_path / "m"), cfg)
    assert w["final.norm"].shape == () and w["l0.mix.q.conv"].shape == (160, 1) and w["side.embed"].shape == (200, 16)


def test_command_line_writes_a_random_model(tmp_path):
    import json
    from nanoinfer_b200.cli import main
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.weights import load_weights
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(tr.R1))
    assert main(["random-model", "--config", str(cfg_file), "--layers", "3", "--seed", "4", "--out", str(tmp_path / "m")]) == 0
    cfg = load_config(str(tmp_path / "m"))
    assert len(cfg.layers) == 3 and cfg.schedule[2].cache_of == 0
    assert set(load_weights(str(tmp_path / "m"), cfg)) >= {"embed", "side.embed", "l2.mix.uk", "final.norm", "head"}


def test_sinusoid_and_convolution_by_hand():
    pe = sinusoid([0, 3], 6, torch.float64)
    assert torch.allclose(pe[0], torch.tensor([0., 1., 0., 1., 0., 1.], dtype=torch.float64))
    f = [1.0, 10000.0 ** (-2 / 6), 10000.0 ** (-4 / 6)]
    want = torch.tensor([v for x in f for v in (torch.sin(torch.tensor(3 * x)), torch.cos(torch.tensor(3 * x)))])
    assert torch.allclose(pe[1], want.double())
    x = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    y, hist = short_conv(x, torch.tensor([[0.5, 10.0, 100.0]], dtype=torch.float64), torch.zeros(2, 1, dtype=torch.float64))
    assert y[:, 0].tolist() == [100.0, 210.0, 320.5] and hist[:, 0].tolist() == [2.0, 3.0]


@pytest.mark.parametrize("raw, seed", [(tr.R1, 1), (tr.R3, 3)])
def test_plain_prompt_equals_token_by_token(tmp_path, raw, seed):
    tr.write_model(str(tmp_path / "m"), raw, seed)
    cfg, w = load_plain(str(tmp_path / "m"))
    model = PlainRunevik(cfg, w)
    toks = random_tokens(cfg["vocab"], 21, seed)
    st = model.new_state()
    whole, _ = model.run(toks, st)
    st = model.new_state()
    parts = [model.run(toks[:9], st)[0], model.run(toks[9:11], st)[0]] + [model.run([t], st)[0] for t in toks[11:]]
    assert torch.allclose(torch.cat(parts), whole, rtol=1e-9, atol=1e-9)
    assert whole.abs().max() > 0.5 and torch.isfinite(whole).all()
