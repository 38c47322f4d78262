"""A plain, slow implementation of the Vuvalorn design, written from its equations: one function per
mechanism, float64, one token after the other, lists for caches.  It shares no code with the package.

Notation: x the stream [width]; h a sublayer's input; H query heads, G key heads, D the head size.

  embedding      x = E[token] * embedding.scale
  layer          x += N1b(mixer(N1(x)));  x += N2b(ff(N2(x)))  (ff may be absent);  N(v) = v / sqrt(mean(v^2) + eps) * w
  loop           layers start .. stop-1 run `times` times; pass t begins with x += loop.step[t]; every pass has
                 caches of its own
  mixer          u_q = W_q h, u_k = W_k h;  c_t = sum_j w[:, j] u_(t - taps + 1 + j)  (zeros before the start);
                 value = c_k;  q, k = N_head(c_q), N_head(c_k);  first rot.dims dimensions rotated in pairs
                 (2i, 2i+1) by the angle p * base^(-2i / dims);  s = q.k * scale, s = cap * tanh(s / cap);
                 softmax over keys 0 .. p;  head h reads key head h // (H / G);  result * sigmoid(W_g h)_h;  W_o
  dense ff       g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit);  W_down (g * sigmoid(1.702 g) * (u + 1))
  routed ff      s = softmax(W_router h);  the `top` largest of s + correction are chosen;  sum of s_e * expert_e(h),
                 expert_e(h) = W_down (silu(W_gate h) * (W_up h)) for e < experts, h itself for the identity experts
  output         logits = E N_final(x) * logit_scale
"""
import math

import torch

F64 = torch.float64


def rms_norm(v, w, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w


def short_conv(history, u, w):
    """history: the inputs before u, oldest first (fewer than taps - 1 near the start); w [channels, taps].
    Returns the output for u; the caller appends u to the history."""
    taps = w.shape[1]
    past = list(history)[-(taps - 1):] if taps > 1 else []
    rows = [torch.zeros_like(u)] * (taps - 1 - len(past)) + past + [u]
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + w[:, j] * rows[j]
    return out


def rotate_pairs(v, position, dims, base):
    """v [heads, D]: the first ``dims`` dimensions of every head, in pairs (2i, 2i + 1)."""
    out = v.clone()
    for i in range(dims // 2):
        a = position * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        out[:, 2 * i] = v[:, 2 * i] * c - v[:, 2 * i + 1] * s
        out[:, 2 * i + 1] = v[:, 2 * i + 1] * c + v[:, 2 * i] * s
    return out


def capped(s, cap):
    return cap * torch.tanh(s / cap) if cap else s


def attend(q, keys, values, scale, cap):
    """q [H, D]; keys, values [n, G, D] (all visible keys): returns [H, D]."""
    n_heads, n_kv = q.shape[0], keys.shape[1]
    out = torch.zeros_like(q)
    for h in range(n_heads):
        g = h // (n_heads // n_kv)
        s = capped((keys[:, g] @ q[h]) * scale, cap)
        p = torch.softmax(s, 0)
        out[h] = p @ values[:, g]
    return out


def capped_unit(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(w_gate @ h, max=limit)
    u = torch.clamp(w_up @ h, -limit, limit)
    return w_down @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def route(h, w_router, correction, top):
    """(chosen experts in the order of their choice scores, all scores)."""
    s = torch.softmax(w_router @ h, 0)
    choice = s + correction
    return torch.topk(choice, top).indices.tolist(), s


def routed_unit(h, w_router, correction, experts, top):
    """experts: list of (w_gate, w_up, w_down); router outputs beyond them are identity experts."""
    chosen, s = route(h, w_router, correction, top)
    out = torch.zeros_like(h)
    for e in chosen:
        if e >= len(experts):
            out = out + s[e] * h
        else:
            w_gate, w_up, w_down = experts[e]
            a = w_gate @ h
            out = out + s[e] * (w_down @ (a * torch.sigmoid(a) * (w_up @ h)))
    return out


def layer_runs(cfg):
    """[(layer, pass number or None)] in the order of execution."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


class PlainVuvalorn:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: v.to(F64) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.runs = layer_runs(cfg)

    def new_state(self):
        """Per run: the keys and values so far and the two convolutions' inputs; and the position."""
        return {"pos": 0, "runs": [{"k": [], "v": [], "uq": [], "uk": []} for _ in self.runs]}

    def mixer(self, i, h, position, st):
        w, m = self.w, self.cfg["layers"][i]["mixer"]
        p = f"l{i}.mix."
        n_heads, n_kv, dim = m["heads"], m["kv_heads"], m["dim"]
        uq, uk = w[p + "q"] @ h, w[p + "k"] @ h
        cq = short_conv(st["uq"], uq, w[p + "q.conv"])
        ck = short_conv(st["uk"], uk, w[p + "k.conv"])
        st["uq"].append(uq)
        st["uk"].append(uk)
        q = rms_norm(cq.view(n_heads, dim), w[p + "q.norm"], self.eps)
        k = rms_norm(ck.view(n_kv, dim), w[p + "k.norm"], self.eps)
        rot = m.get("rot")
        if rot and rot["dims"]:
            q = rotate_pairs(q, position, rot["dims"], rot["base"])
            k = rotate_pairs(k, position, rot["dims"], rot["base"])
        st["k"].append(k)
        st["v"].append(ck.view(n_kv, dim))
        out = attend(q, torch.stack(st["k"]), torch.stack(st["v"]), m["scale"], m.get("softcap"))
        gate = torch.sigmoid(w[p + "g"] @ h)
        return w[p + "o"] @ (out * gate[:, None]).reshape(-1)

    def feed_forward(self, i, h):
        w, mlp = self.w, self.cfg["layers"][i]["mlp"]
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return capped_unit(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["limit"])
        r = mlp["router"]
        experts = [(w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"]) for e in range(r["experts"])]
        return routed_unit(h, w[p + "router"], w[p + "correction"], experts, r["top"])

    def token(self, tok, state, streams=None):
        cfg, w, eps = self.cfg, self.w, self.eps
        x = w["embed"][tok] * (cfg.get("embedding") or {}).get("scale", 1.0)
        for r, (i, t) in enumerate(self.runs):
            if t is not None:
                x = x + w["loop.step"][t]
            p = f"l{i}."
            x = x + rms_norm(self.mixer(i, rms_norm(x, w[p + "norm1"], eps), state["pos"], state["runs"][r]),
                             w[p + "norm1b"], eps)
            if cfg["layers"][i].get("mlp") is not None:
                x = x + rms_norm(self.feed_forward(i, rms_norm(x, w[p + "norm2"], eps)), w[p + "norm2b"], eps)
            if streams is not None:
                streams.append(x.clone())
        state["pos"] += 1
        return (w["embed"] @ rms_norm(x, w["final.norm"], eps)) * cfg.get("logit_scale", 1.0)

    def run(self, tokens, state):
        """Logits [len(tokens), vocab] of the next tokens of the sequence that ``state`` holds."""
        return torch.stack([self.token(int(t), state) for t in tokens])


def whole_sequence(cfg, weights, tokens):
    """The same design once more, for a whole sequence at once in matrices (no caches, no state): what the
    token-by-token form must agree with.  Returns logits [T, vocab]."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    n = len(tokens)
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))

    def conv(u, cw):
        taps = cw.shape[1]
        padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F64), u])
        return sum(padded[j:j + n] * cw[:, j] for j in range(taps))

    def rotate(v, rot):
        if not rot or not rot["dims"]:
            return v
        dims = rot["dims"]
        ang = torch.arange(n, dtype=F64)[:, None] * rot["base"] ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        out = v.clone()
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
        return out

    for i, t in layer_runs(cfg):
        if t is not None:
            x = x + w["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        m = layer["mixer"]
        n_heads, n_kv, dim = m["heads"], m["kv_heads"], m["dim"]
        h = rms_norm(x, w[p + "norm1"], eps)
        cq, ck = conv(h @ w[p + "mix.q"].T, w[p + "mix.q.conv"]), conv(h @ w[p + "mix.k"].T, w[p + "mix.k.conv"])
        q = rotate(rms_norm(cq.view(n, n_heads, dim), w[p + "mix.q.norm"], eps), m.get("rot"))
        k = rotate(rms_norm(ck.view(n, n_kv, dim), w[p + "mix.k.norm"], eps), m.get("rot"))
        v = ck.view(n, n_kv, dim)
        gate = torch.sigmoid(h @ w[p + "mix.g"].T)
        heads = []
        for hd in range(n_heads):
            g = hd // (n_heads // n_kv)
            s = capped((q[:, hd] @ k[:, g].T) * m["scale"], m.get("softcap")).masked_fill(~causal, -math.inf)
            heads.append((torch.softmax(s, -1) @ v[:, g]) * gate[:, hd:hd + 1])
        x = x + rms_norm(torch.cat(heads, -1) @ w[p + "mix.o"].T, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = torch.stack([capped_unit(r, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], mlp["limit"]) for r in h])
            else:
                r_ = mlp["router"]
                experts = [(w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"]) for e in range(r_["experts"])]
                y = torch.stack([routed_unit(r, w[p + "mlp.router"], w[p + "mlp.correction"], experts, r_["top"]) for r in h])
            x = x + rms_norm(y, w[p + "norm2b"], eps)
    return (rms_norm(x, w["final.norm"], eps) @ w["embed"].T) * cfg.get("logit_scale", 1.0)
