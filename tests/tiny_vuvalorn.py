"""Small Vuvalorn configurations for the tests, as config.json dictionaries, and a writer of model folders with
random weights that the tests may tune.

V1 mixes everything: three layers with different head counts, head sizes, taps and rotated shares; a capped
unit, a routed one with an identity expert, a layer without feed-forward; a looped span in the middle.
V2 has sizes the tensor-core attention kernels take (heads of 64, four query heads per key head), no identity
experts, a span of one layer that starts the model and runs three times, and neither scale.
V3 has values that are 1 or absent elsewhere: one head, one tap (no history), no rotation, no cap, top 1, more
identity experts than real ones, no loop, a head size of 128 with five taps.
V4 has sizes that are no multiple of 8 anywhere.
"""
import json
import os

import torch


def attention(heads, kv_heads, dim, conv, rot, scale, cap, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if cap is not None:
        m["softcap"] = cap
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, identity, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


V1 = {"architecture": "Vuvalorn", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
      "logit_scale": 0.7, "loop": {"start": 1, "stop": 3, "times": 2},
      "layers": [attention(4, 2, 24, 3, (12, 10000.0), 0.3, 2.5, dense(136, 0.8)),
                 attention(3, 3, 32, 2, (32, 50000.0), 0.25, 4.0, moe(5, 1, 2, 40)),
                 attention(2, 1, 40, 4, (8, 100.0), 0.2, 3.0, None),
                 attention(4, 2, 24, 3, (24, 10000.0), 0.3, 2.0, moe(6, 2, 3, 24))]}
V2 = {"architecture": "Vuvalorn", "vocab": 260, "width": 128, "norm": {"eps": 1e-6},
      "loop": {"start": 0, "stop": 1, "times": 3},
      "layers": [attention(8, 2, 64, 4, (64, 500000.0), 0.18, 6.0, moe(8, 0, 3, 64)),
                 attention(8, 2, 64, 2, (32, 10000.0), 0.18, 3.0, dense(192, 1.5))]}
V3 = {"architecture": "Vuvalorn", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
      "logit_scale": 2.0,
      "layers": [attention(1, 1, 16, 1, None, 0.4, None, moe(2, 3, 1, 32)),
                 attention(2, 1, 128, 5, (2, 3.0), 0.12, 1.5, dense(64, 0.3))]}
V4 = {"architecture": "Vuvalorn", "vocab": 173, "width": 76, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
      "logit_scale": 0.37, "loop": {"start": 0, "stop": 2, "times": 2},
      "layers": [attention(5, 5, 20, 2, (10, 777.0), 0.33, 2.2, moe(3, 1, 2, 12)),
                 attention(3, 1, 36, 3, (36, 10000.0), 0.2, 5.0, dense(52, 1.1))]}

# Standard deviations that make every mechanism matter in a random model: projections whose results are of order
# one, convolution taps that all count, routers that choose firmly (so that few choices hang on a rounding), output projections and output norms
# that weigh as much as the stream.
LIVELY = {"weight": 0.5, "q": 0.1, "k": 0.1, "g": 0.15, "o": 0.1, "q.conv": 0.5, "k.conv": 0.5, "gate": 0.12, "up": 0.12,
          "down": 0.1, "router": 0.4, "correction": 0.05}


def tune_norms(tensors):
    """Gains that differ from one, so that a norm left out, or the wrong gain, shows."""
    for name, t in tensors.items():
        if name.split(".")[-1] in ("norm1", "norm2", "norm1b", "norm2b", "norm") and t.dim() == 1:
            g = torch.Generator().manual_seed(len(name) * 131 + t.numel())
            t.copy_((1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype))
        if name == "loop.step":
            t.mul_(8.0)


def write_model(model_dir, raw, seed, slot_std=None, tune=None, dtype=torch.bfloat16):
    """config.json + model.safetensors with random weights (the package's own generator and writer);
    ``tune(tensors)`` may change them before they are written.  Returns {name: tensor}."""
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.random_init import random_tensors
    from nanoinfer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    std = dict(LIVELY if slot_std is None else slot_std)
    for p in __import__("nanoinfer_b200.weights.plan", fromlist=["tensor_plan"]).tensor_plan(cfg):
        leaf = p.slot.split(".")[-1]                      # an expert's "e3.gate" is drawn like "gate"
        if p.slot not in std and leaf in std and p.slot[0] == "e":
            std[p.slot] = std[leaf]
    tensors = dict(random_tensors(cfg, seed, 0.05, dtype, std))
    tune_norms(tensors)
    if tune is not None:
        tune(tensors)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors.items())
    return tensors
