"""Vuvalorn without a GPU: the configuration parser, the tensor list, refusals, random model folders, and the plain
implementation against itself (a whole sequence in matrices against the same tokens one by one through caches)."""
import copy

import pytest
import torch

import tiny_vuvalorn as tv
from helpers import load_plain, random_tokens
from plain_vuvalorn import PlainVuvalorn, layer_runs, short_conv, whole_sequence


def test_config_becomes_parts_and_schedule():
    from nanoinfer_b200.config import config_from_dict
    cfg = config_from_dict(tv.V1)
    assert cfg.architecture == "Vuvalorn" and cfg.hidden_size == 96 and cfg.vocab_size == 300
    assert [l.mixer.kind for l in cfg.layers] == ["conv_key_attention"] * 4
    assert [l.feed_forward.kind if l.feed_forward else None for l in cfg.layers] == \
        ["capped_glu", "routed_experts", None, "routed_experts"]
    assert [(r.layer, r.stream_input) for r in cfg.schedule] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert [(r.layer, r.stream_input) for r in cfg.schedule] == [(i, t) for i, t in layer_runs(tv.V1)]
    assert cfg.stream_inputs == 2 and all(r.cache_of is None for r in cfg.schedule)
    m = cfg.layers[2].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.softmax_scale) == (2, 1, 40, 0.2)
    assert m.extra_dict() == {"conv_taps": 4, "norm_eps": 1e-5, "score_cap": 3.0}
    assert m.position.kind == "rope_exact" and m.position.rotary_dim == 8 and m.position.pairing == "interleaved"
    assert cfg.layers[2].ffn_norm is None and cfg.layers[2].ffn_post_norm is None and cfg.layers[2].mixer_post_norm is not None
    assert all(l.arrangement == "sandwich_norm" for l in cfg.layers)
    f = cfg.layers[3].feed_forward.extra_dict()
    assert (f["experts"], f["identity_experts"], f["top"], f["renormalize"]) == (6, 2, 3, False)
    assert cfg.layers[0].feed_forward.extra_dict()["limit"] == 0.8
    assert cfg.embedding.extra_dict()["row_scale"] == 3.0 and cfg.head_spec().tied and cfg.head.extra_dict()["logit_scale"] == 0.7
    plain = config_from_dict(tv.V3)       # no loop, no scales, no rotation, no cap
    assert plain.stream_inputs == 0 and [r.layer for r in plain.schedule] == [0, 1]
    assert plain.layers[0].mixer.position.kind == "none" and plain.layers[0].mixer.extra_dict()["score_cap"] == 0.0
    assert config_from_dict(tv.V2).embedding.extra_dict()["row_scale"] == 1.0


def test_tensor_names_and_shapes():
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.plan import tensor_plan
    plan = {p.name: p.shape for p in tensor_plan(config_from_dict(tv.V1))}
    assert plan["embed"] == (300, 96) and plan["final.norm"] == (96,) and plan["loop.step"] == (2, 96)
    assert "head" not in plan and "lm_head" not in plan
    assert plan["l0.mix.q"] == (96, 96) and plan["l0.mix.k"] == (48, 96) and plan["l0.mix.q.conv"] == (96, 3)
    assert plan["l0.mix.k.conv"] == (48, 3) and plan["l0.mix.q.norm"] == (24,) and plan["l0.mix.k.norm"] == (24,)
    assert plan["l0.mix.g"] == (4, 96) and plan["l0.mix.o"] == (96, 96) and "l0.mix.v" not in plan
    assert plan["l0.mlp.gate"] == (136, 96) and plan["l0.mlp.down"] == (96, 136)
    assert plan["l1.mlp.router"] == (6, 96) and plan["l1.mlp.correction"] == (6,)
    assert plan["l1.mlp.e4.up"] == (40, 96) and plan["l1.mlp.e4.down"] == (96, 40) and "l1.mlp.e5.up" not in plan
    assert all(plan[f"l2.{n}"] == (96,) for n in ("norm1", "norm1b")) and "l2.norm2" not in plan and "l2.norm2b" not in plan
    assert plan["l3.norm2b"] == (96,) and plan["l3.mlp.router"] == (8, 96)
    assert "loop.step" not in {p.name for p in tensor_plan(config_from_dict(tv.V3))}


@pytest.mark.parametrize("change, message", [
    (lambda r: r["layers"][1].update(type="delta"), "not a mixer"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"].update(vdim=16), "values are the keys"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=13), "even"),
    (lambda r: r["layers"][0]["mixer"].update(conv=0), "taps"),
    (lambda r: r["layers"][0]["mlp"].update(kind="polynorm"), "not supported"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda r: r["loop"].update(stop=7), "does not fit"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.pop("width"), "width"),
])
def test_bad_configs_are_refused(change, message):
    from nanoinfer_b200.config import ConfigError, config_from_dict
    raw = copy.deepcopy(tv.V1)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_random_model_folder_round_trip(tmp_path):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.weights import load_weights
    from nanoinfer_b200.weights.loader import WeightError
    d = str(tmp_path / "m")
    written = tv.write_model(d, tv.V4, seed=3)
    cfg = load_config(d)
    w = load_weights(d, cfg)
    assert set(w) == set(written) and all(torch.equal(w[k], written[k]) for k in w)
    raw, plain = load_plain(d)
    assert raw == tv.V4 and plain["l0.mlp.e2.down"].shape == (76, 12)
    # a tensor too many and one missing are both reported
    from nanoinfer_b200.weights.safetensors_io import write_safetensors
    import os
    written["l0.mix.v"] = torch.zeros(4, 4, dtype=torch.bfloat16)
    del written["loop.step"]
    write_safetensors(os.path.join(d, "model.safetensors"), written.items())
    with pytest.raises(WeightError) as e:
        load_weights(d, cfg)
    assert "l0.mix.v" in str(e.value) and "loop.step" in str(e.value)


def test_short_conv_reads_zeros_before_the_start():
    w = torch.tensor([[1.0, 10.0, 100.0], [2.0, 20.0, 200.0]], dtype=torch.float64)
    hist = []
    outs = []
    for t in range(4):
        u = torch.tensor([t + 1.0, -(t + 1.0)], dtype=torch.float64)
        outs.append(short_conv(hist, u, w))
        hist.append(u)
    assert outs[0].tolist() == [100.0, -200.0]                   # only the token's own tap
    assert outs[1].tolist() == [210.0, -420.0]
    assert outs[3].tolist() == [2 + 30 + 400.0, -(4 + 60 + 800.0)]


@pytest.mark.parametrize("raw", [tv.V1, tv.V2, tv.V3, tv.V4], ids=["v1", "v2", "v3", "v4"])
def test_token_by_token_equals_whole_sequence(tmp_path, raw):
    d = str(tmp_path / "m")
    tv.write_model(d, raw, seed=5)
    cfg, w = load_plain(d)
    toks = random_tokens(raw["vocab"], 37, 9)
    plain = PlainVuvalorn(cfg, w)
    st = plain.new_state()
    by_token = torch.cat([plain.run(toks[:20], st), plain.run(toks[20:], st)])
    torch.testing.assert_close(by_token, whole_sequence(cfg, w, toks), rtol=1e-9, atol=1e-9)
    assert by_token.abs().max() > 0.5 and by_token.std() > 0.05          # the model says something


def test_every_mechanism_matters(tmp_path):
    """Leaving out any one mechanism of the plain model moves its logits far beyond rounding: the tests that
    compare the package with it would see the same omission in the package."""
    d = str(tmp_path / "m")
    tv.write_model(d, tv.V1, seed=7)
    cfg, w = load_plain(d)
    toks = random_tokens(300, 40, 2)
    ref = whole_sequence(cfg, w, toks)
    scale = ref.std().item()

    def moved(cfg2, w2):
        return (whole_sequence(cfg2, w2, toks) - ref).pow(2).mean().sqrt().item() / scale

    def cfg_with(fn):
        c = copy.deepcopy(cfg)
        fn(c)
        return c

    def w_with(fn):
        w2 = {k: v.clone() for k, v in w.items()}
        fn(w2)
        return w2

    assert moved(cfg_with(lambda c: c["layers"][0]["mixer"].pop("softcap")), w) > 0.01
    assert moved(cfg_with(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=24)), w) > 0.01
    assert moved(cfg_with(lambda c: c["layers"][0]["mlp"].update(limit=50.0)), w) > 0.01
    assert moved(cfg_with(lambda c: c["loop"].update(times=1)), w) > 0.01
    assert moved(cfg_with(lambda c: c.update(logit_scale=1.0)), w) > 0.01
    assert moved(cfg, w_with(lambda x: x["loop.step"].zero_())) > 0.01
    assert moved(cfg, w_with(lambda x: x["l1.mlp.correction"].zero_())) > 0.001
    assert moved(cfg, w_with(lambda x: x["l0.mix.q.conv"][:, :-1].zero_())) > 0.01
    assert moved(cfg, w_with(lambda x: x["l0.mix.k.conv"][:, 0].zero_())) > 0.01
    assert moved(cfg, w_with(lambda x: x["l0.mix.g"].zero_())) > 0.01
    assert moved(cfg, w_with(lambda x: x["l0.norm1b"].fill_(1.0))) > 0.01
    assert moved(cfg, w_with(lambda x: x["l0.mix.k.norm"].fill_(1.0))) > 0.01
