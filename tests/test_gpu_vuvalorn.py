"""Vuvalorn on the GPU against the plain implementation (tests/plain_vuvalorn.py): every mechanism alone, then
whole models replayed under four ways of cutting the same requests - in 32-bit and in bfloat16 - and greedy
generation through the engine.  The models are small, of other sizes than any real one, with weights tuned so
that a lost key, a lost convolution tap, a missing cap or a wrong expert moves the logits far beyond rounding."""
import json
import os
import subprocess
import sys

import pytest
import torch

import replay_util as ru
import tiny_vuvalorn as tv
from helpers import load_plain, random_tokens
from plain_vuvalorn import (PlainVuvalorn, attend, capped_unit, rms_norm, rotate_pairs, route, routed_unit, short_conv,
                            whole_sequence)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
CUTS = {"whole": ru.whole, "tail": ru.tail_by_token, "ragged": ru.ragged, "mixed": ru.mixed}
LENGTHS = {"v1": [1, 2, 17, 33, 70, 130, 49], "v2": [3, 16, 64, 150, 31, 97], "v3": [2, 48, 129, 15, 80],
           "v4": [5, 1, 66, 23, 90]}
RAW = {"v1": tv.V1, "v2": tv.V2, "v3": tv.V3, "v4": tv.V4}
F64 = torch.float64


def _lone_choice_margin(cfg, w, toks):
    """The smallest gap between the best and the second-best choice score over all positions and all routed layers
    that choose ONE expert (there a choice that a rounding turns over replaces the whole output); 1 if none."""
    plain = PlainVuvalorn(cfg, w)
    worst = [1.0]
    orig = plain.feed_forward

    def watched(i, h):
        mlp = cfg["layers"][i]["mlp"]
        if mlp["kind"] == "moe" and mlp["router"]["top"] == 1:
            p = f"l{i}.mlp."
            best = torch.topk(torch.softmax(plain.w[p + "router"] @ h, 0) + plain.w[p + "correction"], 2).values
            worst[0] = min(worst[0], (best[0] - best[1]).item())
        return orig(i, h)

    plain.feed_forward = watched
    plain.run(toks, plain.new_state())
    return worst[0]


def _requests(cfg, w, vocab, lengths, seed):
    """Random requests; where a layer chooses one expert, a request is drawn again until no choice in it hangs on
    less than 0.03 (bfloat16 rounding moves a choice score by a few thousandths)."""
    reqs = {}
    for i, n in enumerate(lengths):
        for attempt in range(200):
            toks = random_tokens(vocab, n, seed + i + 1000 * attempt)
            if _lone_choice_margin(cfg, w, toks) >= 0.03:
                break
        else:
            raise AssertionError("no request without a close call was found")
        reqs[f"q{i}"] = toks
    return reqs


def _sensitivity(cfg, w, reqs, want):
    """How much more than the median position each position's logits move when every weight is disturbed at the
    size of a bfloat16 rounding: {(request, position): factor >= 1}.  Where a router's choice hangs on little, or
    a sublayer's output is small before it is divided by its root mean square, a position can be many times as
    sensitive as most."""
    g = torch.Generator().manual_seed(0)
    moved = {}
    for trial in range(3):                       # a position's sensitivity depends on the direction: the largest of three
        shaken = {k: v.double() * (1 + 2.0 ** -8 * (torch.rand(v.shape, generator=g, dtype=torch.float64) - 0.5))
                  for k, v in w.items()}
        for rid, toks in reqs.items():
            out = whole_sequence(cfg, shaken, toks).float()
            rel = (out - want[rid]).pow(2).mean(1).sqrt() / want[rid].pow(2).mean(1).sqrt()
            for pos in range(len(toks)):
                moved[(rid, pos)] = max(moved.get((rid, pos), 0.0), rel[pos].item())
    median = sorted(moved.values())[len(moved) // 2]
    return {k: max(1.0, v / (3.0 * median)) for k, v in moved.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{key: (folder, config dictionary, requests, plain logits per request, sensitivity per position)}"""
    root = tmp_path_factory.mktemp("vuvalorn")
    out = {}
    for seed, (key, raw) in enumerate(RAW.items()):
        d = str(root / key)
        tv.write_model(d, raw, seed + 21)
        cfg, w = load_plain(d)
        reqs = _requests(cfg, w, raw["vocab"], LENGTHS[key], 37 * seed)
        want = {rid: whole_sequence(cfg, w, toks).float() for rid, toks in reqs.items()}
        out[key] = (d, cfg, reqs, want, _sensitivity(cfg, w, reqs, want))
    return out


# bfloat16 bounds of the whole-model replays.  A layer of this design rounds often on the way to the stream, and
# every sublayer's output is divided by its own root mean square, so the roundings of a small output count in
# full; and a routed layer may choose another expert where two choice scores are close.  Hence the rule: per
# position twice the bounds of the Llama replays (ru.compare), at most 3 % of the positions over them and none
# over four times, and the bound of a position that is more than three times as sensitive as the median position
# (measured on the plain model, see _sensitivity) grows in proportion.  A lost key, tap, cap or expert moves these
# models' logits by more than that at most positions (the one-layer tests, which keep the tight bounds, show it).
BF16_MAX_REL, BF16_RMS_REL, BF16_SHARE_OVER, BF16_WORST = 0.10, 0.03, 0.03, 4.0


def _compare(got, want, dtype, label, sensitivity=None):
    if dtype == "float32":
        return ru.compare(got, want, dtype, label)
    assert got
    ratios = {}
    for (rid, pos), row in got.items():
        ref = want[rid][pos]
        err = (row - ref).abs()
        ratios[(rid, pos)] = max(err.max().item() / (BF16_MAX_REL * ref.abs().max().item()),
                                 err.pow(2).mean().sqrt().item() / (BF16_RMS_REL * ref.pow(2).mean().sqrt().item())) \
            / (sensitivity or {}).get((rid, pos), 1.0)
    over = {k: round(v, 2) for k, v in ratios.items() if v > 1.0}
    worst = max(ratios.values())
    assert worst <= BF16_WORST, f"{label}: worst position at {worst:.2f} times the bound: {over}"
    assert len(over) <= max(1, BF16_SHARE_OVER * len(ratios)), f"{label}: {len(over)} of {len(ratios)} positions over the bound: {over}"


def _runner(model_dir, dtype, steps, page=16, max_requests=4, **kw):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights
    cfg = load_config(model_dir)
    num_pages = max(1, ru.max_live_tokens(steps, 64) // page)
    return ModelRunner(cfg, load_weights(model_dir, cfg), dtype=dtype, page_size=page, num_pages=num_pages,
                       max_requests=max_requests, **kw)


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


# ---- mechanisms alone ---------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rowwise_kernels(dtype):
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    tol = _tol(dtype)
    # scaled embedding, odd width, an id out of range
    table = torch.randn(50, 37, generator=g).to(dtype)
    toks = torch.tensor([3, 49, 0, 77, 12], dtype=torch.int32)
    out = torch.empty(5, 37, dtype=torch.float32, device=DEV)
    ops.embedding_scaled(toks.to(DEV), table.to(DEV), 2.5, out)
    want = table.float()[toks.clamp(max=49).long()] * 2.5
    want[3] = 0
    torch.testing.assert_close(out.cpu(), want, rtol=1e-6, atol=1e-6)
    # a row added to every token of the stream
    h = torch.randn(7, 37, generator=g)
    row = torch.randn(37, generator=g)
    hd = h.to(DEV)
    ops.add_row(hd, row.to(DEV))
    torch.testing.assert_close(hd.cpu(), h + row, rtol=1e-6, atol=1e-6)
    # scaling in place
    x = torch.randn(3, 41, generator=g)
    xd = x.to(DEV)
    ops.scale_f32(xd, 0.37)
    torch.testing.assert_close(xd.cpu(), x * 0.37, rtol=1e-6, atol=1e-7)
    # the capped unit's activation, values on both sides of the limit
    gu = (torch.randn(9, 2 * 26, generator=g) * 2).to(dtype)
    act = torch.empty(9, 26, dtype=dtype, device=DEV)
    ops.capped_glu(gu.to(DEV), act, 0.9, 1.702, 1.0)
    gf, uf = gu.float()[:, :26].clamp(max=0.9), gu.float()[:, 26:].clamp(-0.9, 0.9)
    assert (gu.float()[:, :26] > 0.9).any() and (gu.float()[:, 26:] < -0.9).any() and (gu.float()[:, :26] < -0.9).any()
    torch.testing.assert_close(act.float().cpu(), gf * torch.sigmoid(1.702 * gf) * (uf + 1.0), **tol)


@pytest.mark.parametrize("H, G, D, taps, rot", [(4, 2, 24, 3, 12), (5, 5, 20, 2, 10), (1, 1, 160, 1, 0), (2, 1, 128, 5, 128),
                                                (3, 1, 36, 4, 36), (2, 2, 64, 6, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_norm_rotation_and_cache_write(H, G, D, taps, rot, dtype):
    """Three requests in one launch: a fresh one, one that goes on at a position past a page border with a
    history, one with a single token (a portion shorter than the history); slots out of order; extra columns
    behind the channels.  Queries, key pages, value pages and the new histories against the plain functions."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(H * 100 + D + taps)
    page, base, eps = 8, 700.0, 1e-5
    C = (H + G) * D
    starts, lens, slots = [0, 21, 9], [11, 6, 1], [2, 0, 3]
    n = sum(lens)
    proj = torch.randn(n, C + H, generator=g).to(dtype)
    conv_w = torch.randn(C, taps, generator=g) * 0.5
    qg, kg = 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    state = torch.randn(4, (taps - 1) * C, generator=g).to(dtype).float()       # values a projection could have left
    state[2] = 0                                                               # the fresh request's slot
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)] or [0.0], dtype=torch.float32)
    positions = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lens)]).int()
    seq_of = torch.repeat_interleave(torch.arange(3), torch.tensor(lens)).int()
    cu = torch.tensor([0, 11, 17, 18], dtype=torch.int32)
    table = torch.tensor([[5, 1, 9, 0], [3, 8, 2, 6], [7, 4, 0, 0]], dtype=torch.int32)
    k_pages = torch.zeros(10, G, page, D, dtype=dtype, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    q_out = torch.empty(n, H * D, dtype=dtype, device=DEV)
    state_d = state.to(DEV)
    ops.conv_qk_prepare(proj.to(DEV), conv_w.t().contiguous().to(DEV), qg.to(DEV), kg.to(DEV), eps, state_d, positions.to(DEV),
                        seq_of.to(DEV), cu.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV), 3, table.to(DEV),
                        inv_freq.to(DEV), q_out, k_pages, v_pages, H, G, D, rot, taps, page)
    tol = _tol(dtype)
    row = 0
    for s, (start, ln, slot) in enumerate(zip(starts, lens, slots)):
        hist = [state[slot].double().view(taps - 1, C)[r] for r in range(taps - 1)] if taps > 1 else []
        for i in range(ln):
            u = proj[row, :C].double()
            c = short_conv(hist, u, conv_w.double())
            hist.append(u)
            pos = start + i
            q = rms_norm(c[:H * D].view(H, D), qg.double(), eps)
            k = rms_norm(c[H * D:].view(G, D), kg.double(), eps)
            if rot:
                q, k = rotate_pairs(q, pos, rot, base), rotate_pairs(k, pos, rot, base)
            torch.testing.assert_close(q_out[row].double().cpu().view(H, D), q, **tol)
            pg = table[s, pos // page].item()
            torch.testing.assert_close(k_pages[pg, :, pos % page].double().cpu(), k, **tol)
            torch.testing.assert_close(v_pages[pg, :, pos % page].double().cpu(), c[H * D:].view(G, D), **tol)
            row += 1
        if taps > 1:
            want = torch.stack(hist[-(taps - 1):]).reshape(-1)
            torch.testing.assert_close(state_d[slot].double().cpu(), want, rtol=0, atol=0)      # copied, not computed
    assert torch.equal(state_d[1].cpu(), state[1])                                               # nobody's slot


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq, Hkv, D, cap", [(4, 2, 24, 2.0), (3, 1, 96, 5.0), (8, 2, 64, 3.0), (4, 1, 128, 1.5)])
def test_attention_with_capped_scores(dtype, Hq, Hkv, D, cap):
    """Scores far beyond the cap on some keys: without the cap those keys would take all the weight."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(D + Hq)
    page, n_keys = 16, 83
    k = torch.randn(n_keys, Hkv, D, generator=g)
    k[5] *= 6.0
    k[70] *= 6.0
    v = torch.randn(n_keys, Hkv, D, generator=g)
    q = torch.randn(3, Hq, D, generator=g)
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    pos = [n_keys - 1, 40, 6]
    perm = [3, 0, 5, 1, 4, 2]
    k_pages = torch.zeros(6, Hkv, page, D, dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    for j in range(n_keys):
        k_pages[perm[j // page], :, j % page] = k[j]
        v_pages[perm[j // page], :, j % page] = v[j]
    out = torch.empty(3, Hq * D, dtype=dtype, device=DEV)
    table = torch.tensor([perm] * 3, dtype=torch.int32, device=DEV)
    ops.attention_generic(q.view(3, -1).to(DEV), k_pages.to(DEV), v_pages.to(DEV), out,
                          torch.tensor(pos, dtype=torch.int32, device=DEV), torch.arange(3, dtype=torch.int32, device=DEV),
                          table, Hq, Hkv, D, page, None, 0.3, score_cap=cap)
    for i, p in enumerate(pos):
        want = attend(q[i].double(), k[:p + 1].double(), v[:p + 1].double(), 0.3, cap)
        free = attend(q[i].double(), k[:p + 1].double(), v[:p + 1].double(), 0.3, None)
        torch.testing.assert_close(out[i].double().cpu().view(Hq, D), want, **_tol(dtype))
        assert (want - free).abs().max() > 0.05


@pytest.mark.parametrize("Hq, Hkv, D, cap", [(8, 2, 64, 3.0), (4, 1, 128, 1.5), (6, 3, 96, 4.0), (2, 2, 64, 2.0), (3, 1, 128, 6.0)])
def test_tensor_core_attention_with_capped_scores(Hq, Hkv, D, cap):
    """The bfloat16 kernels for prompt portions (mma.sync) and for single tokens (split over the keys) take the
    cap too: portions of 300 and 150 tokens behind contexts of 0 and 77, and single tokens at contexts of 1 to
    700, against the plain kernel (which the test above holds against the plain implementation)."""
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.mixer import PagedAttendMixin
    g = torch.Generator().manual_seed(D * Hq)
    bf, i32, page = torch.bfloat16, torch.int32, 16
    n_pages = 100
    k_pages = torch.randn(n_pages, Hkv, page, D, generator=g).to(bf).to(DEV)
    k_pages[:, :, 3] *= 5.0                            # keys whose raw scores lie far beyond the cap
    v_pages = torch.randn(n_pages, Hkv, page, D, generator=g).to(bf).to(DEV)
    perm = torch.randperm(n_pages, generator=g).int()

    def run(q_lens, starts):
        n = sum(q_lens)
        q = torch.randn(n, Hq * D, generator=g).to(bf).to(DEV)
        kv = [a + b for a, b in zip(q_lens, starts)]
        width = max(-(-x // page) for x in kv)
        table = torch.zeros(len(q_lens), width, dtype=i32)
        at = 0
        for i, x in enumerate(kv):
            need = -(-x // page)
            table[i, :need] = perm[at:at + need]
            at += need
        pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, q_lens)]).int().to(DEV)
        seq = torch.repeat_interleave(torch.arange(len(q_lens)), torch.tensor(q_lens)).int().to(DEV)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=i32, device=DEV)
        table = table.to(DEV)
        want = torch.empty_like(q)
        ops.attention_generic(q, k_pages, v_pages, want, pos, seq, table, Hq, Hkv, D, page, None, 0.11, score_cap=cap)
        free = torch.empty_like(q)
        ops.attention_generic(q, k_pages, v_pages, free, pos, seq, table, Hq, Hkv, D, page, None, 0.11)
        assert (want.float() - free.float()).abs().max() > 0.05, "the cap must bite"
        got = torch.empty_like(q)
        if max(q_lens) == 1:
            if D not in ops.DECODE_HEAD_DIMS:
                return
            splits = ops.decode_splits(n, Hkv, D, max(kv))
            scratch = torch.empty(n * Hq * splits * (D + 2), dtype=torch.float32, device=DEV)
            tickets = torch.zeros(n * Hkv, dtype=i32, device=DEV)
            ops.attention_decode(q, k_pages, v_pages, got, None, n, pos, seq, table, Hq, Hkv, D, page, None, 0.11, splits,
                                 scratch, tickets, score_cap=cap)
        else:
            plan = PagedAttendMixin.plan_step(q_lens, starts)
            ops.attention_prefill(q, k_pages, v_pages, got, torch.from_numpy(plan.arrays["tile_seq"]).to(DEV),
                                  torch.from_numpy(plan.arrays["tile_row0"]).to(DEV), plan.scalars["n_tiles"], cu,
                                  torch.tensor(kv, dtype=i32, device=DEV), table, Hq, Hkv, D, page, None, 0.11, kernel="mma",
                                  score_cap=cap)
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)

    run([300, 150], [0, 77])
    run([1, 1, 1, 1], [0, 15, 256, 699])


@pytest.mark.parametrize("n_real, n_id, top, d, f, n", [(5, 1, 2, 96, 40, 3), (5, 1, 2, 96, 40, 150), (8, 0, 3, 128, 64, 16),
                                                        (2, 3, 1, 64, 32, 70), (3, 1, 2, 76, 12, 40), (0, 2, 1, 64, 8, 9),
                                                        (40, 2, 6, 64, 16, 300), (8, 0, 3, 128, 64, 200), (6, 0, 6, 64, 24, 33), (8, 0, 3, 128, 64, 1),
                                                        (16, 2, 4, 256, 64, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_and_experts(dtype, n_real, n_id, top, d, f, n):
    """The routed part alone: choices and weights against the plain router, the output against the plain unit,
    for a few rows (one warp per output in bfloat16) and for many (pairs laid out expert by expert)."""
    from nanoinfer_b200.config.model_config import FeedForwardSpec
    from nanoinfer_b200.engine.runtime import Runtime
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.feed_forward import RoutedExperts
    g = torch.Generator().manual_seed(n_real * 7 + n)
    spec = FeedForwardSpec(kind="routed_experts", intermediate_size=f,
                           extra=(("experts", n_real), ("identity_experts", n_id), ("top", top), ("choice_bias", True)))
    bf = lambda t: t.to(torch.bfloat16)
    w = {"router": bf(torch.randn(n_real + n_id, d, generator=g) * 0.3), "correction": bf(torch.randn(n_real + n_id, generator=g) * 0.05)}
    for e in range(n_real):
        w[f"e{e}.gate"], w[f"e{e}.up"] = bf(torch.randn(f, d, generator=g) * 0.15), bf(torch.randn(f, d, generator=g) * 0.15)
        w[f"e{e}.down"] = bf(torch.randn(d, f, generator=g) * 0.2)
    rt = Runtime(device=torch.device(DEV), dtype=dtype, page_size=16)
    ops.preload(["routed"])
    part = RoutedExperts(spec, d, w, rt)
    x = torch.randn(n, d, generator=g).to(dtype)
    # router alone
    ids = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
    counts = torch.zeros(max(n_real, 1), dtype=torch.int32, device=DEV)
    ops.route(x.to(DEV), part.w_router, part.bias, ids, wts, counts, n_real, top)
    experts = [(w[f"e{e}.gate"].double(), w[f"e{e}.up"].double(), w[f"e{e}.down"].double()) for e in range(n_real)]
    want_counts = [0] * max(n_real, 1)
    close = []
    for t in range(n):
        chosen, s = route(x[t].double(), w["router"].double(), w["correction"].double(), top)
        c = torch.sort(s + w["correction"].double(), descending=True).values
        close.append(top < n_real + n_id and (c[top - 1] - c[top]).item() < 1e-5)
        if close[-1]:
            continue
        assert ids[t].tolist() == chosen, f"token {t}"
        torch.testing.assert_close(wts[t].double().cpu(), s[chosen], rtol=1e-5, atol=1e-6)
    assert sum(close) <= max(1, n // 50)
    for e in ids.cpu().flatten().tolist():
        if e < n_real:
            want_counts[e] += 1
    assert counts.tolist() == want_counts
    # the whole part; run twice: its counters must be left as they were found
    for _ in range(2):
        y = part.forward(x.to(DEV), None)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=4e-2)
    for t in range(n):
        if not close[t]:
            want = routed_unit(x[t].double(), w["router"].double(), w["correction"].double(), experts, top)
            scale = max(1.0, want.abs().max().item())             # bfloat16 roundings grow with the size of the sums
            torch.testing.assert_close(y[t].double().cpu() / scale, want / scale, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capped_unit_alone(dtype):
    from nanoinfer_b200.config.model_config import FeedForwardSpec
    from nanoinfer_b200.engine.runtime import Runtime
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.feed_forward import CappedGLU
    g = torch.Generator().manual_seed(3)
    d, f = 72, 44
    spec = FeedForwardSpec(kind="capped_glu", intermediate_size=f, extra=(("limit", 0.6), ("gate_slope", 1.702), ("up_shift", 1.0)))
    w = {k: (torch.randn(s, generator=g) * 0.2).to(torch.bfloat16) for k, s in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f)))}
    ops.preload(["pointwise"])
    part = CappedGLU(spec, d, w, Runtime(device=torch.device(DEV), dtype=dtype, page_size=16))
    for n in (2, 50):
        x = torch.randn(n, d, generator=g).to(dtype)
        y = part.forward(x.to(DEV), None)
        want = torch.stack([capped_unit(r.double(), w["gate"].double(), w["up"].double(), w["down"].double(), 0.6) for r in x])
        torch.testing.assert_close(y.double().cpu(), want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32
                                                               else dict(rtol=3e-2, atol=2e-2)))


# ---- one layer, tuned ------------------------------------------------------------------------------------

def _one_layer(layer, width=64, vocab=120, **top):
    raw = {"architecture": "Vuvalorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [layer]}
    raw.update(top)
    return raw


@pytest.mark.parametrize("D", [48, 64, 128])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_a_far_key(tmp_path, dtype, D):
    """Token 4's query points where token 2's key points (one coordinate of the embedding each, which no other
    token has), and nobody else's.  The prompt ends with token 4; token 2 stands only at position 3, hundreds of
    keys back.  With token 3 there instead the logits at the end move by much, and the engine must follow both
    prompts - through portions that end at and just after page borders, then token by token."""
    from nanoinfer_b200.engine import StepEntry

    def tune(t):
        e = t["embed"]
        e[:, 60] = 0
        e[:, 61] = 0
        e[2, 60] = 3.0                                   # what only token 2 has: most of its key
        e[4, 61] = 3.0                                   # what only token 4 has: most of its query
        k, q = t["l0.mix.k"], t["l0.mix.q"]
        k[:, 60] = k[:, 60].sign() * 0.5
        k[:, 61] = 0
        q[:, 60] = 0
        q[:, 61] = torch.cat([k[:, 60], k[:, 60]])       # token 4's query points where token 2's key points
        for name in ("l0.mix.q.conv", "l0.mix.k.conv"):
            t[name][:, :-1] *= 0.05                      # mostly the current token
            t[name][:, -1] = 1.0
        t["l0.mix.q.norm"].fill_(1.0)
        t["l0.mix.k.norm"].fill_(1.0)
        t["l0.mix.g"].zero_()
        t["l0.norm1b"].fill_(6.0)                        # the mixer weighs more than the stream
    n, far = 300, 3
    raw = _one_layer(tv.attention(2, 1, D, 3, (4, 10000.0), 1.2 / D ** 0.5, 10.0, None), embedding={"scale": 4.0})
    d = str(tmp_path / "m")
    tv.write_model(d, raw, 7, tune=tune)
    cfg, w = load_plain(d)
    base = [5 + (i % 90) for i in range(n)]
    base[far], base[-1] = 2, 4
    other = list(base)
    other[far] = 3
    want = {k: whole_sequence(cfg, w, t)[-1].float() for k, t in (("same", base), ("other", other))}
    moved = (want["same"] - want["other"]).abs().max().item()
    assert moved > 0.25 * want["same"].abs().max().item(), "the test's weights do not make the far token count"
    steps = ru.whole({"same": base, "other": other})
    runner = _runner(d, dtype, steps, max_requests=2)
    for k, toks in (("same", base), ("other", other)):
        cuts = [0, 250, 256, 257, 272, 290] + list(range(291, n + 1))
        for a, b in zip(cuts, cuts[1:]):
            logits = runner.step([StepEntry(k, toks[a:b], [b - a - 1])])
        runner.end(k)
        ru.compare({(k, n - 1): logits[0].cpu()}, {k: {n - 1: want[k]}}, dtype, label=f"far key, {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_history_across_portions(tmp_path, dtype):
    """Six taps, every tap weighty: the first five tokens read zeros before the start, and every portion of one to
    four tokens is shorter than the history it needs from the state."""
    def tune(t):
        for name in ("l0.mix.q.conv", "l0.mix.k.conv"):
            t[name].copy_((0.4 + t[name].float().abs()).to(t[name].dtype))
    raw = _one_layer(tv.attention(4, 2, 16, 6, (16, 100.0), 0.3, 3.0, tv.dense(40, 0.7)), logit_scale=1.5)
    d = str(tmp_path / "m")
    tv.write_model(d, raw, 11, tune=tune)
    cfg, w = load_plain(d)
    toks = random_tokens(120, 41, 4)
    want = {"a": whole_sequence(cfg, w, toks).float()}
    sizes = [1, 1, 2, 1, 3, 4, 1, 2, 9, 1, 1, 5, 2, 8]
    steps, at = [], 0
    for i, s in enumerate(sizes):
        steps.append({"step": i, "entries": [{"id": "a", "tokens": toks[at:at + s], "want": list(range(s))}], "end": []})
        at += s
    assert at == len(toks)
    steps[-1]["end"] = ["a"]
    runner = _runner(d, dtype, steps)
    _compare(ru.run_trace(runner, steps), want, dtype, "short portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stream_inputs_between_passes(tmp_path, dtype):
    """A span of two layers that runs three times in the middle of four: with the vectors between the passes
    large, a pass that took another pass's vector, or none, shows at once."""
    def tune(t):
        t["loop.step"].mul_(5.0)
    layers = [tv.attention(2, 2, 16, 2, (8, 50.0), 0.3, 4.0, None), tv.attention(2, 1, 16, 3, (16, 50.0), 0.3, 4.0, tv.dense(32, 1.0)),
              tv.attention(4, 4, 8, 1, None, 0.5, None, tv.moe(3, 1, 2, 16)), tv.attention(1, 1, 32, 2, (32, 50.0), 0.2, 4.0, None)]
    raw = {"architecture": "Vuvalorn", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "layers": layers,
           "loop": {"start": 1, "stop": 3, "times": 3}}
    d = str(tmp_path / "m")
    tv.write_model(d, raw, 13, tune=tune)
    cfg, w = load_plain(d)
    reqs = {"a": random_tokens(90, 45, 1), "b": random_tokens(90, 20, 2)}
    want = {k: whole_sequence(cfg, w, t).float() for k, t in reqs.items()}
    steps = ru.mixed(reqs, tail=5)
    runner = _runner(d, dtype, steps)
    assert len(runner.caches) == 8 and len({id(c.k_pages) for c in runner.caches}) == 8       # a cache per run
    _compare(ru.run_trace(runner, steps), want, dtype, "looped span", sensitivity=_sensitivity(cfg, w, reqs, want))


# ---- whole models, cut in four ways ---------------------------------------------------------------------

@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(RAW))
def test_replay_matches_plain(models, key, dtype, cut):
    """Exactly as many pages as the trace needs and four slots, so both are used again."""
    d, cfg, reqs, want, sens = models[key]
    steps = CUTS[cut](reqs)
    runner = _runner(d, dtype, steps)
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _compare(got, want, dtype, label=f"{key} {cut}", sensitivity=sens)
    runner.cache.check_consistency()
    assert runner.cache.num_free_slots == 4


@pytest.mark.parametrize("key", list(RAW))
def test_float32_does_not_depend_on_the_cut(models, key):
    """In 32-bit every cut gives the same bits: portions, batches, pages and slots only move data."""
    d, cfg, reqs, want, sens = models[key]
    ref = None
    for cut in CUTS:
        steps = CUTS[cut](reqs)
        got = ru.run_trace(_runner(d, "float32", steps), steps)
        if ref is None:
            ref = got
        else:
            for k in ref:
                assert torch.equal(ref[k], got[k]), f"{key}: {cut} differs from whole at {k}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_replayed_graphs(models, dtype):
    """Most of a request token by token (the steps are captured and replayed from the third on), a second request
    decoding beside it from the middle on."""
    d, cfg, reqs, want, sens = models["v2"]
    reqs = {k: reqs[k] for k in ("q3", "q5")}
    steps = ru.tail_by_token({"q3": reqs["q3"]}, tail=140)
    join = ru.tail_by_token({"q5": reqs["q5"]}, tail=60)
    for i, st in enumerate(join):                       # q5 runs beside q3's single tokens
        steps[30 + i]["entries"] += st["entries"]
        steps[30 + i]["end"] += st["end"]
    runner = _runner(d, dtype, steps)
    _compare(ru.run_trace(runner, steps), want, dtype, label="long decoding", sensitivity=sens)
    assert runner._graphs, "no step of single tokens was captured"


def test_greedy_generation_through_the_engine(models):
    """Engine.generate (scheduler, chunked prompts, sampling kernels) against greedy decoding of the plain model."""
    from nanoinfer_b200 import Engine, SamplingParams
    d, cfg, reqs, want, sens = models["v1"]
    raw_cfg, w = load_plain(d)
    plain = PlainVuvalorn(raw_cfg, w)
    prompts = [reqs["q2"], reqs["q3"][:20], reqs["q1"]]
    engine = Engine.from_model_dir(d, dtype="float32", block_size=16, num_cache_blocks=64, max_batch_size=4,
                                   max_sequences=4, prefill_chunk_size=12)
    out = engine.generate(prompts, max_new_tokens=12, sampling_params=SamplingParams.greedy())
    for prompt, got in zip(prompts, out):
        st = plain.new_state()
        logits = plain.run(prompt, st)[-1]
        for t in got:
            top2 = torch.topk(logits, 2).values
            if int(torch.argmax(logits)) != t:
                assert (top2[0] - logits[t]).item() < 1e-4, "the engine chose a token that the plain model ranks lower"
            logits = plain.run([t], st)[-1]
        assert len(got) == 12


def test_trace_replay_from_the_command_line(models, tmp_path):
    """bin/trace_run as a user runs it: the model class follows from config.json."""
    d, cfg, reqs, want, sens = models["v4"]
    reqs = {k: reqs[k] for k in ("q2", "q3")}
    steps = ru.mixed(reqs, tail=4)
    out = str(tmp_path / "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", str(ru.max_live_tokens(steps, 64))], input="\n".join(json.dumps(s) for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, fed = {}, {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        rows = torch.from_file(os.path.join(out, f"{st['step']}.f32"), size=n_want * cfg["vocab"], dtype=torch.float32).view(n_want, -1)
        r = 0
        for e in st["entries"]:
            for wpos in e["want"]:
                got[(e["id"], fed.get(e["id"], 0) + wpos)] = rows[r].clone()
                r += 1
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
    ru.compare(got, want, "float32", "trace_run")
