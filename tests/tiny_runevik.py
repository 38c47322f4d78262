"""Small Runevik configurations for the tests, as config.json dictionaries, and a writer of model folders
with random weights that the tests may tune.

R1 mixes everything: a latent-attention layer, a delta layer with three taps and one key head for two value
heads, a layer that borrows the first layer's latents, a delta layer without feed-forward, token inputs.
R2 has no token inputs, a latent rank (64) and head count that the split-K decode kernel takes, four taps.
R3 has values that are 1 or equal elsewhere: one tap (no convolution history), one head, a latent rank of
128 under two heads (the tcgen05 prompt kernel), a key size above 128.
"""
import json
import os

import torch


def delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent(heads, dim, vdim, rank, scale, ff, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


R1 = {"architecture": "Runevik", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
      "layers": [latent(3, 16, 24, 48, 0.31, 160), delta(2, 1, 24, 40, 3, 136), latent(2, 32, 16, 48, 0.2, 96, kv_from=0),
                 delta(3, 3, 16, 32, 2, 0)]}
R2 = {"architecture": "Runevik", "vocab": 260, "width": 128, "norm": {"eps": 1e-6},
      "layers": [delta(6, 2, 64, 32, 4, 192), latent(4, 32, 32, 64, 0.25, 192), latent(4, 16, 48, 64, 0.4, 0, kv_from=1)]}
R3 = {"architecture": "Runevik", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "token_side": {"dim": 4},
      "layers": [delta(1, 1, 160, 32, 1, 64), latent(2, 16, 16, 128, 0.3, 64), delta(2, 2, 8, 8, 5, 0),
                 latent(1, 24, 40, 128, 0.15, 0, kv_from=1)]}

# Standard deviations that make every mechanism matter in a random model: activation numbers of order one,
# peaked attention (scores with a standard deviation of 1 to 2; sharper ones would pass bfloat16 rounding
# through the exponential at full size), output projections that weigh as much as the stream.
LIVELY = {"act": 0.6, "uk": 0.25, "q": 0.05, "dkv": 0.12, "uv": 0.15, "o": 0.08, "v": 0.1, "k": 0.1, "g": 0.1,
          "up": 0.1, "down": 0.08, "gate": 0.1, "proj": 0.2, "layer_inputs": 0.5, "weight": 0.5, "b": 0.1, "a": 0.1,
          "q.conv": 0.5, "k.conv": 0.5, "v.conv": 0.5, "dt_bias": 0.5, "A_log": 0.5}


def write_model(model_dir, raw, seed, slot_std=None, tune=None, dtype=torch.bfloat16):
    """config.json + model.safetensors with random weights (the package's own generator and writer);
    ``tune(tensors)`` may change them before they are written.  Returns {name: tensor}."""
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.random_init import random_tensors
    from nanoinfer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    tensors = dict(random_tensors(cfg, seed, 0.05, dtype, LIVELY if slot_std is None else slot_std))
    if tune is not None:
        tune(tensors)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors.items())
    return tensors
