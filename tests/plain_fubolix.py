"""A plain, slow statement of the Fubolix decoder: whole sequences, no cache, float64, one function per mechanism.

It shares no code with the package: the configuration is the config.json dictionary and the weights a dictionary of
checkpoint names to tensors.  Every query has its own softmax row over an explicit boolean mask, the sink is an extra
term of the denominator written out as such, and the short convolution is a loop over its taps.
"""

from __future__ import annotations

import math

import torch

F = torch.float64
ROUND = None  # a dtype, or a function of a tensor: activations pass through it wherever a 16-bit pipeline would store them
SINK = True   # False: the softmax without its sink (to show that a test would notice a sink left out)


def r(t):
    """What a reduced-precision pipeline keeps of an activation; the identity unless `ROUND` is set."""
    if ROUND is None:
        return t
    return ROUND(t) if callable(ROUND) else t.to(ROUND).to(F)


def dynamic_tanh(x, w, b, alpha):
    """The norm that takes no statistics: tanh(alpha x) w + b."""
    return torch.tanh(alpha * x) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def relu_squared(z):
    return torch.relu(z) ** 2


def yarn_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies of the dims / 2 pairs, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    sc = rot.get("scaling")
    out = []
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def where(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(where(float(sc["fast"]))), 0)
        hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
        out.append(f)
    return torch.tensor(out, dtype=F), (0.1 * math.log(float(sc["factor"])) + 1.0) if sc else 1.0


def rotate(x, positions, rot: dict, layout: str):
    """x [T, heads, dim]: the first rot.dims features of every head turn by position; `layout` "interleaved" pairs
    (2i, 2i+1), "half" pairs (i, i + dims/2)."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    f, mag = yarn_frequencies(rot)
    ang = positions.to(F)[:, None] * f[None, :]           # [T, dims/2]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - v * sin
        out[..., dims // 2: dims] = v * cos + u * sin
    return out


def causal_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def causal_mask(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def window_mask(T, size, keep_first):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def softmax_with_sink(s, mask, sink):
    """s [H, T, T] scores, mask [T, T]; `sink` [H]: a term exp(sink_h) in every row's denominator that has no value."""
    s = s.masked_fill(~mask[None], -math.inf)
    top = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + (torch.exp(sink[:, None, None] - top) if SINK else 0.0))


def attend(q, k, v, scale, mask, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv]; query head h reads key head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    kk, vv = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk) * scale
    p = softmax_with_sink(s, mask, sink)
    return torch.einsum("hts,shd->thd", p, vv).reshape(T, -1)


def mixer_attention(h, m, W, pre, eps, positions):
    """Keys double as values, interleaved rotation, unit q and k per head after it, window with kept first keys, a sink of
    score 0, a sigmoid gate per head."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = r(h @ W[pre + "q"].T).view(T, H, d)
    k = r(h @ W[pre + "k"].T).view(T, G, d)
    v = k
    q = r(unit_rms(rotate(q, positions, m["rot"], "interleaved"), eps))
    kn = r(unit_rms(rotate(k, positions, m["rot"], "interleaved"), eps))
    mask = window_mask(T, int(m["mask"]["size"]), int(m["mask"].get("keep_first") or 0))
    o = attend(q, kn, v, float(m["scale"]), mask, torch.zeros(H, dtype=F)).view(T, H, -1)
    gate = torch.sigmoid(r(h @ W[pre + "g"].T))                     # [T, H]
    return r(r(o * gate[:, :, None]).reshape(T, -1) @ W[pre + "o"].T)


def mixer_attention_2(h, m, W, pre, eps, positions):
    """q and k normed per head with a gain, no rotation, a query temperature that grows with position, all earlier keys,
    a sink of score 0."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = r(h @ W[pre + "q"].T).view(T, H, d)
    k = r(h @ W[pre + "k"].T).view(T, G, d)
    v = r(h @ W[pre + "v"].T).view(T, G, dv)
    q = unit_rms(q, eps) * W[pre + "q.norm"]
    k = r(unit_rms(k, eps) * W[pre + "k.norm"])
    qt = m.get("q_temp")
    if qt:
        temp = 1.0 + float(qt["coef"]) * torch.log(torch.floor((positions.to(F) + 1.0) / float(qt["every"])) + 1.0)
        q = q * temp[:, None, None]
    q = r(q)
    o = attend(q, k, v, float(m["scale"]), causal_mask(T), torch.zeros(H, dtype=F))
    return r(r(o) @ W[pre + "o"].T)


def mixer_attention_3(h, m, W, pre, eps, positions):
    """A short convolution over time on q, k and v, rotation in halves, all earlier keys, a learned sink per head."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = causal_convolution(r(h @ W[pre + "q"].T), W[pre + "q.conv"]).view(T, H, d)
    k = causal_convolution(r(h @ W[pre + "k"].T), W[pre + "k.conv"]).view(T, G, d)
    v = r(causal_convolution(r(h @ W[pre + "v"].T), W[pre + "v.conv"])).view(T, G, dv)
    q, k = r(rotate(q, positions, m["rot"], "half")), r(rotate(k, positions, m["rot"], "half"))
    o = attend(q, k, v, float(m["scale"]), causal_mask(T), W[pre + "sink"].to(F))
    return r(r(o) @ W[pre + "o"].T)


MIXERS = {"attention": mixer_attention, "attention_2": mixer_attention_2, "attention_3": mixer_attention_3}


def feed_forward(h, W, pre):
    return r(r(relu_squared(r(h @ W[pre + "up"].T))) @ W[pre + "down"].T)


def forward(cfg: dict, weights: dict, tokens, rounded=None, layers_out: list | None = None):
    """tokens: a list of ids of one sequence -> float64 logits [T, vocab].  `layers_out` receives the stream after each layer."""
    global ROUND
    ROUND = rounded
    try:
        W = {k: torch.as_tensor(v).to(F) for k, v in weights.items()}
        eps = float(cfg["norm"]["eps"])
        ids = torch.as_tensor(tokens, dtype=torch.long)
        positions = torch.arange(len(ids))
        x = W["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = r(dynamic_tanh(x, W[p + "norm1"], W[p + "norm1.b"], W[p + "norm1.alpha"]))
            y = MIXERS[layer["type"]](h, layer["mixer"], W, p + "mix.", eps, positions)
            if layer.get("mlp") is not None:
                y = y + feed_forward(h, W, p + "mlp.")
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        h = r(dynamic_tanh(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"]))
        return h @ W["head"].T
    finally:
        ROUND = None
