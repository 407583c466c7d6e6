"""Attention whose cache holds one latent vector per token instead of keys and values per head.

    q      = W_q h                          per head [dim plain | rot_dim rotated]
    [c|kr] = W_dkv h                        c: rank features, RMS-normed with a gain; kr: rot_dim features, a single
                                            rotated key vector that every head uses
    key_h  = [W_uk,h c | kr],  value_h = W_uv,h c
    score  = (q_plain . key_plain + q_rot . kr) * scale,   causal, inside a window when one is set
    softmax, optionally with a learned sink per head in the denominator; optionally head h's output times
    sigmoid((W_g h)_h) (gate "head", W_g [heads, hidden]), or every feature of the heads side by side times the sigmoid
    of its own gate (gate "feature", W_g [heads * v_dim, hidden]); output projection over the heads side by side.

Only [c | kr] is cached (a lane with one key head of rank + rot_dim features and no values).  Keys and values are never
formed: the plain part of the query is folded through W_uk (q_lat = W_uk,h^T q_plain, a product per head), attention runs
over the cached vectors with one shared key head whose first `rank` features are also the value (`ops.attention_latent`),
and the result is unfolded through W_uv,h.  Prompts, portions and single tokens all take this route, so the numbers at a
position do not depend on the cut.  The rotation, the latent's norm, scores, softmax and the gate's sigmoid are float32.

params: hidden, heads, dim, rot_dim, v_dim, rank, scale, window (0: every key), eps (of the latent's norm), sink (bool),
gate (False, True or "head", or "feature"), position (a "rotary" PartSpec over rot_dim features, or None), names (optional: tensor names after the
part's prefix, keys "q", "dkv", "dkv_norm", "uk", "uv", "o", "sink", "g").
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Part, StateNeed, WeightSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part

_DEFAULT_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o", "sink": "sink", "g": "g"}


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.rot_dim, self.v_dim, self.rank = int(p["dim"]), int(p["rot_dim"]), int(p["v_dim"]), int(p["rank"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window") or 0)
        self.eps = float(p["eps"])
        self.has_sink, self.has_gate = bool(p.get("sink")), bool(p.get("gate"))
        self.gate_kind = None if not self.has_gate else "head" if p["gate"] is True else str(p["gate"])
        if self.gate_kind not in (None, "head", "feature"):
            raise ValueError(f"latent attention: unknown gate {self.gate_kind!r} (\"head\" or \"feature\")")
        self.gate_size = 0 if not self.has_gate else self.heads if self.gate_kind == "head" else self.heads * self.v_dim
        self.names = {**_DEFAULT_NAMES, **dict(p.get("names") or {})}
        self.position = build_part("position", p["position"], dtype, device) if p.get("position") is not None else None
        if self.position is not None and (not getattr(self.position, "interleaved", False) or self.position.dims > self.rot_dim):
            raise ValueError("latent attention rotates interleaved pairs of at most rot_dim features")
        self.q_size = self.heads * (self.dim + self.rot_dim)
        self.off_latent = self.q_size
        self.off_gate = self.q_size + self.rank + self.rot_dim
        self.w_proj = self.w_uk = self.w_uk_t = self.w_uv = self.w_o = self.c_gain = self.sink = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        n, H = self.names, self.heads
        specs = {
            n["q"]: WeightSpec((self.q_size, self.hidden)),
            n["dkv"]: WeightSpec((self.rank + self.rot_dim, self.hidden)),
            n["dkv_norm"]: WeightSpec((self.rank,), rule="float32", init="gain"),
            n["uk"]: WeightSpec((H * self.dim, self.rank), std=0.05),
            n["uv"]: WeightSpec((H * self.v_dim, self.rank), std=0.05),
            n["o"]: WeightSpec((self.hidden, H * self.v_dim)),
        }
        if self.has_sink:
            specs[n["sink"]] = WeightSpec((H,), rule="float32", init="normal", std=1.0)
        if self.has_gate:
            specs[n["g"]] = WeightSpec((self.gate_size, self.hidden))
        return specs

    def bind(self, tensors) -> None:
        n, H = self.names, self.heads
        rows = [tensors[n["q"]], tensors[n["dkv"]]] + ([tensors[n["g"]]] if self.has_gate else [])
        w = torch.cat(rows, dim=0)
        extra = -w.shape[0] % 8  # rows of the projection's output start on 16 bytes in bfloat16
        if extra:
            w = torch.cat([w, torch.zeros((extra, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.w_proj = w.contiguous()
        self.w_uk = tensors[n["uk"]].view(H, self.dim, self.rank).contiguous()         # [H, dim, rank]: q_plain @ it
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous()                            # [H, rank, dim]: rows of a product's weight
        self.w_uv = tensors[n["uv"]].view(H, self.v_dim, self.rank).contiguous()       # [H, v_dim, rank]
        self.w_o = tensors[n["o"]].contiguous()
        self.c_gain = tensors[n["dkv_norm"]].contiguous()
        self.sink = tensors[n["sink"]].contiguous() if self.has_sink else None

    def cache_need(self) -> CacheNeed | None:
        return CacheNeed(1, self.rank + self.rot_dim, self.window, 0, 0)

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, x, ctx: StepContext, lane: LaneView, writes: bool = True):
        N, H, R, d, r, dv = ctx.n_tokens, self.heads, self.rank, self.dim, self.rot_dim, self.v_dim
        proj = ctx.buffer("latent_proj", self.w_proj.shape[0])
        ops.linear(x, self.w_proj, proj)
        pos = self.position
        ops.latent_rope_store(proj, ctx, lane, pos.inv_freq if pos is not None and pos.dims else None,
                              pos.magnitude if pos is not None else 1.0, self.c_gain, self.eps, H, d, r, R, write=writes)
        q = proj[:, : self.q_size].unflatten(1, (H, d + r))
        q_plain, q_rot = q[:, :, :d], q[:, :, d:]
        # fold the plain part of every head's query through W_uk: [H, N, R]
        q_lat = ctx.buffer("latent_q", H * R).view(-1)[: H * N * R].view(H, N, R)
        o_lat = ctx.buffer("latent_o", H * R).view(-1)[: H * N * R].view(H, N, R)
        attn = ctx.buffer("attn_out", H * dv)
        if self.dtype == torch.float32:  # the float32 product kernel, a head at a time
            for h in range(H):
                ops.linear(q_plain[:, h, :], self.w_uk_t[h], q_lat[h])
        else:
            torch.bmm(q_plain.permute(1, 0, 2), self.w_uk, out=q_lat)
        gate = proj[:, self.off_gate: self.off_gate + H] if self.gate_kind == "head" else None
        ops.attention_latent(q_lat.permute(1, 0, 2), q_rot, lane, ctx, o_lat.permute(1, 0, 2), self.scale, self.window,
                             self.sink, gate)
        if self.dtype == torch.float32:
            for h in range(H):
                ops.linear(o_lat[h], self.w_uv[h], attn[:, h * dv: (h + 1) * dv])
        else:
            torch.bmm(o_lat, self.w_uv.transpose(1, 2), out=attn.view(N, H, dv).permute(1, 0, 2))
        if self.gate_kind == "feature":
            ops.sigmoid_mul(attn, proj[:, self.off_gate: self.off_gate + H * dv])
        return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden))
