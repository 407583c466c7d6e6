"""A plain, slow statement of the Debuvik decoder: whole sequences, no cache, float64, one function per mechanism.

It shares no code with the package: the configuration is the config.json dictionary and the weights a dictionary of
checkpoint names to tensors.  Keys and values of the latent layers are decompressed per head, every query has its own
softmax row over an explicit mask, and a layer that borrows another layer's keys reads them from a dictionary of
what the lending layer formed.
"""

from __future__ import annotations

import math

import torch

F = torch.float64
ROUND = None  # a dtype, or a function of a tensor: activations pass through it wherever a 16-bit pipeline would store them (`forward(..., rounded=)`)


def r(t):
    """What a reduced-precision pipeline keeps of an activation; the identity unless `ROUND` is set."""
    if ROUND is None:
        return t
    return ROUND(t) if callable(ROUND) else t.to(ROUND).to(F)


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def banded_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims), then the wavelength bands: short waves stay, long waves turn `factor` times slower, the
    band between is blended."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < original / high:
                pass
            elif wave > original / low:
                f = f / factor
            else:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate_half(x, positions, rot: dict | None):
    """x [T, heads, n]: feature i of the first rot.dims features is paired with feature i + dims/2; the rest pass."""
    if not rot or int(rot["dims"]) == 0:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    ang = positions.to(F)[:, None] * banded_frequencies(rot)[None, :]      # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def chunk_mask(T: int, size: int | None) -> torch.Tensor:
    """mask[i, j]: j <= i and, with a chunk size, both in the same chunk counted from the start of the sequence."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i // size == j // size)
    return ok


def softmax_rows(scores, mask):
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)


def latent_attention(h, w: dict, m: dict, eps: float):
    """h [T, width]; `w`: the mixer's tensors by their short names; `m`: the layer's "mixer" block."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = r(h @ w["q"].T).view(T, H, d)
    c = r(rms_norm(r(h @ w["dkv"].T), w["dkv.norm"], eps))                  # [T, rank]
    k = r(c @ w["uk"].T).view(T, H, d)
    v = r(c @ w["uv"].T).view(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    p = softmax_rows(scores, chunk_mask(T, None))
    o = r(torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * dv))
    o = r(o * torch.sigmoid(r(h @ w["g"].T)))
    return r(o @ w["o"].T)


def attention_keys(h, w: dict, m: dict, eps: float, positions):
    """The keys (normed over the whole projection, rotated) and values a layer forms: ([T, G, d], [T, G, dv])."""
    T = h.shape[0]
    G, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = rms_norm(r(h @ w["k"].T) + w["k.b"], w["k.norm"], eps).view(T, G, d)
    v = r(r(h @ w["v"].T) + w["v.b"]).view(T, G, dv)
    return r(rotate_half(k, positions, m.get("rot"))), v


def attention(h, w: dict, m: dict, eps: float, positions, kv):
    """`kv`: (keys, values) of this layer or of the layer it borrows them from."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_norm(r(h @ w["q"].T) + w["q.b"], w["q.norm"], eps).view(T, H, d)
    q = r(rotate_half(q, positions, m.get("rot")))
    k, v = kv
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        scores = float(cap) * torch.tanh(scores / float(cap))
    p = softmax_rows(scores, chunk_mask(T, int((m.get("mask") or {}).get("size") or 0) or None))
    o = r(torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * dv))
    return r(o @ w["o"].T) + w["o.b"]


def dense_ff(h, w: dict):
    return r(r(silu(r(h @ w["gate"].T)) * r(h @ w["up"].T)) @ w["down"].T)


def token_side(x, tokens, table, i: int, dim: int, w: dict, eps: float):
    """The layer's own slice of a second embedding, gated by the stream, projected back and normed."""
    e = table[tokens][:, i * dim: (i + 1) * dim]
    g = r(gelu_tanh(r(x @ w["gate"].T)) * e)
    return rms_norm(r(g @ w["proj"].T), w["norm"], eps)


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F) for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, layers_out: list | None = None, rounded=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `layers_out`, when given, receives the stream after every layer.
    `rounded`: a dtype through which the activations pass wherever a pipeline of that type would store them (the stream
    itself, norms, scores and softmax stay exact), or a function that stands for such a storage: how far rounding alone moves
    the result."""
    global ROUND
    before, ROUND = ROUND, rounded
    try:
        return _forward(cfg, weights, tokens, layers_out)
    finally:
        ROUND = before


def _forward(cfg: dict, weights: dict, tokens, layers_out: list | None) -> torch.Tensor:
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    eps = float(cfg["norm"]["eps"])
    x = weights["embed"].to(F)[tokens]
    side = cfg.get("token_side")
    formed: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        w = sub(weights, p + "mix.")
        if layer["type"] == "latent_attention":
            y = latent_attention(r(x), w, m, eps)
        elif layer["type"] == "attention":
            if m.get("kv_from") is None:
                formed[i] = attention_keys(r(x), w, m, eps, positions)
            y = attention(r(x), w, m, eps, positions, formed[i if m.get("kv_from") is None else int(m["kv_from"])])
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, weights[p + "norm1"].to(F), eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(r(x), sub(weights, p + "mlp.")), weights[p + "norm2"].to(F), eps)
        if side:
            x = x + token_side(r(x), tokens, weights["side.embed"].to(F), i, int(side["dim"]), sub(weights, p + "side."), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = r(rms_norm(x, weights["final.norm"].to(F), eps))
    return x @ weights["head"].to(F).T
