"""Grouped-query attention over the paged cache (the reference's `Attention`,
model/llama.py:161-184): packed q/k/v projection without bias, position encoding of q and
k, the step's keys and values written to their pages, softmax(q k^T / sqrt(d)) v over every
key at or before the query's position (and inside the window, if one is set), output
projection.  Query head h reads kv head h // (heads / kv_heads).

Interface of a mixer part:
    cache_need() -> CacheNeed | None      paged storage wanted per token
    state_need() -> StateNeed | None      fixed-size state wanted per request
    forward(x, ctx, lane, writes) -> y    x, y: [N, hidden] in the compute dtype
A mixer may also take part in folding the norms into its products (`Part.takes_row_scaled`,
`Part.feeds_norm_sink`); this one does.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheNeed, Part, StateNeed, WeightSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


@register_part("mixer", "gqa_attention")
class GQAAttention(Part):
    """params: hidden, heads, kv_heads, head_dim, window (0 = all keys), position (PartSpec),
    scale (optional; default 1/sqrt(head_dim)); and, all optional:
    v_dim        the values' head size when it is not the keys' (the output projection then takes heads * v_dim)
    keep_first   with a window: the first so many keys of a sequence stay visible to every later query
    qk_norm      {"eps": e}: an RMS norm over the whole q projection and one over the whole k projection (one statistic
                 over all heads, gains `q_norm` / `k_norm` of the projections' sizes), before the rotation
    wide_weights True: the softmax weights keep about 16 bits where they meet the values (`ops.attention`)
    chunk        c > 0: the sequence is cut into chunks of c positions counted from the start of the sequence and a query sees only the
                 keys of its own chunk (at or before its position)
    softcap      c > 0: a scaled score s becomes c * tanh(s / c) before the softmax
    bias         True: q, k, v and o have biases (float32 in every mode; names "q_bias", "k_bias", "v_bias", "o_bias",
                 default the weight's name + ".b"); the q/k/v biases are added before the q/k norm
    own_kv       False: the mixer has no k and v projections (nor their norm and biases): it reads the lane that another
                 layer's mixer of the same head counts, sizes and rotation writes (the recipe gives it a run with
                 `writes=False` on that lane), with queries, mask and output projection of its own
    names        the tensors' names after the part's prefix, keys "q", "k", "v", "o", "q_norm", "k_norm"
                 (default the Hugging Face ones)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot be shared among {self.kv_heads} kv heads")
        self.v_dim = int(p.get("v_dim") or self.head_dim)
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.qk_norm = dict(p["qk_norm"]) if p.get("qk_norm") else None
        self.wide_weights = bool(p.get("wide_weights"))
        self.chunk = int(p.get("chunk") or 0)
        self.softcap = float(p.get("softcap") or 0.0)
        self.has_bias = bool(p.get("bias"))
        self.own_kv = bool(p.get("own_kv", True))
        if self.chunk and self.keep_first:
            raise ValueError("kept first keys and chunks do not go together")
        names = dict(p.get("names") or {})
        self.names = {k: names.get(k, d) for k, d in (("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"),
                                                      ("o", "o_proj.weight"), ("q_norm", "q_norm.weight"), ("k_norm", "k_norm.weight"))}
        for k in ("q", "k", "v", "o"):
            self.names[k + "_bias"] = names.get(k + "_bias", self.names[k] + ".b")
        self.q_size = self.heads * self.head_dim
        self.kv_size = self.kv_heads * self.head_dim
        self.v_size = self.kv_heads * self.v_dim
        self.o_in = self.heads * self.v_dim
        # what the llama-shaped fast paths (a projection with the rotation in its epilogue) do not know of
        self.general = self.v_dim != self.head_dim or self.qk_norm is not None or self.has_bias or not self.own_kv
        self.qkv_bias: torch.Tensor | None = None
        self.o_bias: torch.Tensor | None = None
        self.q_gain: torch.Tensor | None = None
        self.k_gain: torch.Tensor | None = None
        self.position = build_part("position", p["position"], dtype, device) if p.get("position") is not None else None
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        n = self.names
        specs = {n["q"]: WeightSpec((self.q_size, self.hidden)), n["o"]: WeightSpec((self.hidden, self.o_in))}
        if self.own_kv:
            specs[n["k"]] = WeightSpec((self.kv_size, self.hidden))
            specs[n["v"]] = WeightSpec((self.v_size, self.hidden))
        if self.qk_norm is not None:
            specs[n["q_norm"]] = WeightSpec((self.q_size,), rule="float32", init="gain")
            if self.own_kv:
                specs[n["k_norm"]] = WeightSpec((self.kv_size,), rule="float32", init="gain")
        if self.has_bias:
            sizes = {"q": self.q_size, "k": self.kv_size, "v": self.v_size, "o": self.hidden}
            for k in ("q", "k", "v", "o") if self.own_kv else ("q", "o"):
                specs[n[k + "_bias"]] = WeightSpec((sizes[k],), rule="float32", init="normal")
        return specs

    def bind(self, tensors) -> None:
        n = self.names
        kinds = ("q", "k", "v") if self.own_kv else ("q",)
        # one packed projection [q | k | v]: one matrix product instead of three
        self.w_qkv = torch.cat([tensors[n[k]] for k in kinds], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.qk_norm is not None:
            self.q_gain = tensors[n["q_norm"]].contiguous()
            self.k_gain = tensors[n["k_norm"]].contiguous() if self.own_kv else None
        if self.has_bias:
            self.qkv_bias = torch.cat([tensors[n[k + "_bias"]] for k in kinds], dim=0).contiguous()
            self.o_bias = tensors[n["o_bias"]].contiguous()

    def cache_need(self) -> CacheNeed | None:
        # (a chunked mask keeps every page: a layer that reads this lane may be masked otherwise)
        return CacheNeed(self.kv_heads, self.head_dim, self.window, self.keep_first,
                         None if self.v_dim == self.head_dim else self.v_dim)

    def state_need(self) -> StateNeed | None:
        return None

    def takes_row_scaled(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_qkv)

    def feeds_norm_sink(self, n_tokens: int) -> bool:
        return self.o_bias is None and ops.norm_fusion_ok(n_tokens, self.dtype, self.w_o)

    @property
    def branch_bias(self) -> torch.Tensor | None:
        """The output projection's bias: an arrangement that norms the branch in a kernel of its own may call
        `forward(..., leave_bias=True)` and add this there."""
        return self.o_bias

    def forward(self, x, ctx: StepContext, lane: LaneView, writes: bool = True, sink: ops.NormSink | None = None,
                leave_bias: bool = False):
        qkv = ctx.buffer("qkv", self.w_qkv.shape[0])
        if self.general:
            ops.linear(x, self.w_qkv, qkv)
            if self.position is None:
                raise ValueError("an attention mixer with qk_norm, v_dim, biases or borrowed keys takes a position part with the "
                                 "general rotate_and_store")
            if not self.own_kv and writes:
                raise ValueError("an attention mixer without k and v projections reads a lane that another run writes")
            qn = self.qk_norm
            extra = {"bias": self.qkv_bias} if self.qkv_bias is not None else {}
            self.position.rotate_and_store(qkv, ctx, lane, self.heads, self.kv_heads if self.own_kv else 0, self.head_dim, writes,
                                           v_dim=self.v_dim, q_gain=self.q_gain, k_gain=self.k_gain,
                                           eps=float(qn["eps"]) if qn else 0.0, **extra)
            attn = ctx.buffer("attn_out", self.o_in)
            ops.attention(qkv, lane, ctx, attn, self.heads, self.kv_heads, self.head_dim, self.scale, self.window,
                          self.keep_first, self.v_dim, self.wide_weights, self.chunk, self.softcap)
            if self.o_bias is not None and leave_bias:
                return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden))
            if self.o_bias is not None:
                return ops.add_bias(ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden)), self.o_bias)
            return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden), sink=sink)
        fused = getattr(self.position, "project_rotate_store", None)
        if fused is None or not fused(x, self.w_qkv, qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim, writes):
            ops.linear(x, self.w_qkv, qkv)
            if self.position is not None:
                self.position.rotate_and_store(qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim, writes)
            elif writes:
                ops.kv_store(qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim)
        attn = ctx.buffer("attn_out", self.q_size)
        ops.attention(qkv, lane, ctx, attn, self.heads, self.kv_heads, self.head_dim, self.scale, self.window, self.keep_first,
                      wide_weights=self.wide_weights, chunk=self.chunk, softcap=self.softcap)
        return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden), sink=sink)
