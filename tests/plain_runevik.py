"""A plain, slow implementation of the Runevik design for the tests: one function per mechanism,
written from the design's equations with torch on the CPU, sharing no code with the package.

Everything runs in one floating-point type (float64 by default), token by token where the design
is recurrent, so it is the yardstick and not a model of the package's roundings.

Notation: d = model width, T = tokens of one sequence, p = position (from 0).
"""
import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def over_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def sinusoid(positions, width, dtype):
    """Pairs (sin, cos) of the angles p * f_j, f_j = 10000^(-2j / width), interleaved along the width."""
    out = torch.zeros(len(positions), width, dtype=dtype)
    p = torch.as_tensor(positions, dtype=dtype)[:, None]
    i = torch.arange((width + 1) // 2, dtype=dtype)[None, :]
    ang = p * torch.pow(torch.tensor(10000.0, dtype=dtype), -2.0 * i / width)
    out[:, 0::2] = torch.sin(ang)[:, :out[:, 0::2].shape[1]]
    out[:, 1::2] = torch.cos(ang)[:, :out[:, 1::2].shape[1]]
    return out


def short_conv(x, taps_w, history):
    """Causal convolution over time per channel.  x [T, C]; taps_w [C, K] (last column = current
    token); history [K-1, C] = the inputs before x (zeros at a sequence's start).
    Returns (y [T, C], new history)."""
    k = taps_w.shape[1]
    full = torch.cat([history, x], dim=0)                      # [K-1+T, C]
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        window = full[t:t + k]                                 # inputs t-K+1 .. t
        y[t] = (window * taps_w.t()).sum(dim=0)
    return y, full[full.shape[0] - (k - 1):] if k > 1 else full[:0]


def delta_state(m, dtype):
    chans = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
    return {"S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=dtype),
            "hist_q": torch.zeros(m["conv"] - 1, m["kv_heads"] * m["dim"], dtype=dtype),
            "hist_k": torch.zeros(m["conv"] - 1, m["kv_heads"] * m["dim"], dtype=dtype),
            "hist_v": torch.zeros(m["conv"] - 1, m["heads"] * m["vdim"], dtype=dtype), "chans": chans}


def delta_mixer(h, w, m, eps, st):
    """Gated delta rule over the tokens h [T, d] of one sequence, carrying st."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, st["hist_q"] = short_conv(h @ w["q"].t(), w["q.conv"], st["hist_q"])
    k, st["hist_k"] = short_conv(h @ w["k"].t(), w["k.conv"], st["hist_k"])
    v, st["hist_v"] = short_conv(h @ w["v"].t(), w["v.conv"], st["hist_v"])
    q, k, v = silu(q).view(T, G, D), silu(k).view(T, G, D), silu(v).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].t())                                         # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].t() + w["dt_bias"]))
    gate = silu(h @ w["g"].t()).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    S = st["S"]
    per = H // G
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // per], q[t, hd // per]
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].t() @ kk)
            S[hd] = S[hd] + torch.outer(kk, u)
            out[t, hd] = S[hd].t() @ qq
    out = over_rms(out, eps) * w["norm"] * gate
    return out.reshape(T, H * V) @ w["o"].t()


def latent_of(h, w, eps):
    """The cached latent of each token: RMS norm (plain weight) of W_dkv h."""
    return over_rms(h @ w["dkv"].t(), eps) * w["dkv.norm"]


def latent_attention(h, w, m, eps, latents, start):
    """h [T, d]: tokens at positions start .. start+T-1; latents [start+T, R]: every token's latent
    so far (this layer's own or the one it borrows).  Causal softmax attention per head."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].t()).view(T, H, D)
    keys = (latents @ w["uk"].t()).view(-1, H, D)
    vals = (latents @ w["uv"].t()).view(-1, H, V)
    gate = torch.sigmoid(h @ w["g"].t())                                         # [T, H]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        n = start + t + 1
        for hd in range(H):
            s = (keys[:n, hd] @ q[t, hd]) * m["scale"]
            p = torch.softmax(s, dim=0)
            out[t, hd] = (p[:, None] * vals[:n, hd]).sum(0) * gate[t, hd]
    return out.reshape(T, H * V) @ w["o"].t()


def polynorm_ff(h, w, eps):
    z = h @ w["up"].t()
    a, b, c, e = w["act"]
    act = a * over_rms(z, eps) + b * over_rms(z ** 2, eps) + c * over_rms(z ** 3, eps) + e
    return act @ w["down"].t()


def token_side(x, tokens, layer, side_dim, side_embed, w, eps):
    e = side_embed[tokens, layer * side_dim:(layer + 1) * side_dim]
    y = (gelu_tanh(x @ w["gate"].t()) * e) @ w["proj"].t()
    return x + over_rms(y, eps) * w["norm"]


class PlainRunevik:
    """raw: the config.json dictionary; weights: {tensor name: tensor}.  ``new_state()`` makes the
    state of one sequence; ``run(tokens, state)`` feeds its next tokens and returns
    (logits [T, vocab], residual stream after every layer [L, T, d])."""

    def __init__(self, raw, weights, dtype=torch.float64):
        self.raw, self.dtype = raw, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.eps = float(raw["norm"]["eps"])
        self.side = raw.get("token_side")

    def sub(self, prefix):
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        st = {"n": 0, "layers": []}
        for layer in self.raw["layers"]:
            if layer["type"] == "delta":
                st["layers"].append(delta_state(layer["mixer"], self.dtype))
            else:
                st["layers"].append({"latents": torch.zeros(0, layer["mixer"]["kv_rank"], dtype=self.dtype)})
        return st

    def run(self, tokens, st):
        raw, eps, d = self.raw, self.eps, self.raw["width"]
        tokens = torch.as_tensor(tokens, dtype=torch.long)
        start, T = st["n"], len(tokens)
        x = self.w["embed"][tokens] + sinusoid(range(start, start + T), d, self.dtype)
        after = []
        for i, layer in enumerate(raw["layers"]):
            m = layer["mixer"]
            h = over_rms(x, eps) * self.w[f"l{i}.norm1"]
            mw = self.sub(f"l{i}.mix.")
            if layer["type"] == "delta":
                y = delta_mixer(h, mw, m, eps, st["layers"][i])
            elif layer["type"] == "latent_attention":
                if m.get("kv_from") is None:
                    own = st["layers"][i]
                    own["latents"] = torch.cat([own["latents"], latent_of(h, mw, eps)], dim=0)
                    lat = own["latents"]
                else:
                    lat = st["layers"][m["kv_from"]]["latents"]
                y = latent_attention(h, mw, m, eps, lat, start)
            else:
                raise ValueError(layer["type"])
            if layer.get("mlp") is not None:
                y = y + polynorm_ff(h, self.sub(f"l{i}.mlp."), eps)
            x = x + y
            if self.side is not None:
                x = token_side(x, tokens, i, self.side["dim"], self.w["side.embed"], self.sub(f"l{i}.side."), eps)
            after.append(x.clone())
        st["n"] = start + T
        logits = (over_rms(x, eps) * self.w["final.norm"]) @ self.w["head"].t()
        return logits, torch.stack(after)
