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
    sink         "zero": the softmax's denominator holds one more term, exp(0) = 1, that has no key and no value; "learned": that term
                 is exp(sink[h]) with a float32 tensor of one number per head (name "sink"); default none
    names        the tensors' names after the part's prefix, keys "q", "k", "v", "o", "q_norm", "k_norm"
                 (default the Hugging Face ones).
    The next five act on one head at a time and run in one kernel between the projection and the attention (`ops.head_prepare_store`);
    with any of them the position part is a "rotary" one or None, and `qk_norm`, `bias` and `own_kv=False` are not available:
    head_norm    {"eps": e, "when": "before" | "after", "gain": bool}: an RMS norm of every q head and every k head over its own
                 features, before or after the rotation, with gains `q_norm` / `k_norm` of head_dim entries shared by the heads, or none
    q_temp       {"coef": c, "every": n}: the queries at position p are multiplied by 1 + c * ln(floor((p + 1) / n) + 1)
    head_gate    True: a projection `g` of one row per head; head h's output is multiplied by sigmoid(g(x)[h]) before `o`
    v_from_k     True: no v projection; the values are the keys as projected, before norm and rotation
    conv         taps > 0: q, k and v pass a causal convolution over time per channel right after the projection (tensors `q_conv`,
                 `k_conv`, `v_conv` [channels, taps], float32, default names the projections' + ".conv"); the last taps - 1 projected
                 rows of a request are kept in a state slot (`state_need`), beside the paged keys and values."""

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
        self.sink_kind = p.get("sink")
        if self.sink_kind not in (None, "zero", "learned"):
            raise ValueError(f"gqa_attention: sink {self.sink_kind!r} (None, 'zero' or 'learned')")
        self.head_norm = dict(p["head_norm"]) if p.get("head_norm") else None
        self.q_temp = dict(p["q_temp"]) if p.get("q_temp") else None
        self.head_gate = bool(p.get("head_gate"))
        self.v_from_k = bool(p.get("v_from_k"))
        self.taps = int(p.get("conv") or 0)
        self.per_head = bool(self.head_norm or self.q_temp or self.head_gate or self.v_from_k or self.taps)
        if self.per_head and (self.qk_norm is not None or self.has_bias or not self.own_kv):
            raise ValueError("gqa_attention: head_norm, q_temp, head_gate, v_from_k and conv do not go with qk_norm, bias or borrowed keys")
        if self.head_norm and self.head_norm.get("when", "before") not in ("before", "after"):
            raise ValueError(f"gqa_attention: head_norm.when {self.head_norm.get('when')!r} ('before' or 'after' the rotation)")
        if self.v_from_k and self.v_dim != self.head_dim:
            raise ValueError(f"gqa_attention: keys that double as values have one width, not {self.head_dim} and {self.v_dim}")
        if self.chunk and self.keep_first:
            raise ValueError("kept first keys and chunks do not go together")
        names = dict(p.get("names") or {})
        self.names = {k: names.get(k, d) for k, d in (("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"),
                                                      ("o", "o_proj.weight"), ("q_norm", "q_norm.weight"), ("k_norm", "k_norm.weight"))}
        for k in ("q", "k", "v", "o"):
            self.names[k + "_bias"] = names.get(k + "_bias", self.names[k] + ".b")
        for k in ("q", "k", "v"):
            self.names[k + "_conv"] = names.get(k + "_conv", self.names[k] + ".conv")
        self.names["g"], self.names["sink"] = names.get("g", "g_proj.weight"), names.get("sink", "sink")
        self.q_size = self.heads * self.head_dim
        self.kv_size = self.kv_heads * self.head_dim
        self.v_size = self.kv_heads * self.v_dim
        self.o_in = self.heads * self.v_dim
        # what the llama-shaped fast paths (a projection with the rotation in its epilogue) do not know of
        self.general = self.v_dim != self.head_dim or self.qk_norm is not None or self.has_bias or not self.own_kv
        # the packed projection's columns on the per-head path: [q | k | v (unless the keys double as values) | g (the heads' gates)]
        self.channels = self.q_size + self.kv_size + (0 if self.v_from_k else self.v_size)
        self.sink: torch.Tensor | None = None
        self.conv_taps: torch.Tensor | None = None
        self.qkv_bias: torch.Tensor | None = None
        self.o_bias: torch.Tensor | None = None
        self.q_gain: torch.Tensor | None = None
        self.k_gain: torch.Tensor | None = None
        self.position = build_part("position", p["position"], dtype, device) if p.get("position") is not None else None
        if self.per_head and self.position is not None and not hasattr(self.position, "magnitude"):
            raise ValueError("gqa_attention: the per-head steps take a \"rotary\" position part (frequencies, pairing, magnitude) or none")
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        n = self.names
        specs = {n["q"]: WeightSpec((self.q_size, self.hidden)), n["o"]: WeightSpec((self.hidden, self.o_in))}
        if self.own_kv:
            specs[n["k"]] = WeightSpec((self.kv_size, self.hidden))
            if not self.v_from_k:
                specs[n["v"]] = WeightSpec((self.v_size, self.hidden))
        if self.head_norm and self.head_norm.get("gain"):
            specs[n["q_norm"]] = WeightSpec((self.head_dim,), rule="float32", init="gain")
            specs[n["k_norm"]] = WeightSpec((self.head_dim,), rule="float32", init="gain")
        if self.head_gate:
            specs[n["g"]] = WeightSpec((self.heads, self.hidden))
        if self.sink_kind == "learned":
            specs[n["sink"]] = WeightSpec((self.heads,), rule="float32", init="normal", std=1.0)
        if self.taps:
            sizes = {"q": self.q_size, "k": self.kv_size, "v": self.v_size}
            for k in ("q", "k") if self.v_from_k else ("q", "k", "v"):
                specs[n[k + "_conv"]] = WeightSpec((sizes[k], self.taps), rule="float32", init="normal", std=0.5)
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
        kinds = (("q", "k") if self.v_from_k else ("q", "k", "v")) if self.own_kv else ("q",)
        # one packed projection [q | k | v]: one matrix product instead of three
        self.w_qkv = torch.cat([tensors[n[k]] for k in kinds + (("g",) if self.head_gate else ())], dim=0).contiguous()
        if self.per_head and self.w_qkv.shape[0] % 8:  # rows of the product start on 16 bytes in bfloat16
            pad = torch.zeros((-self.w_qkv.shape[0] % 8, self.hidden), dtype=self.w_qkv.dtype, device=self.w_qkv.device)
            self.w_qkv = torch.cat([self.w_qkv, pad], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.head_norm and self.head_norm.get("gain"):
            self.q_gain, self.k_gain = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()
        if self.sink_kind == "learned":
            self.sink = tensors[n["sink"]].contiguous()
        elif self.sink_kind == "zero":
            self.sink = torch.zeros(self.heads, dtype=torch.float32, device=self.w_o.device)
        if self.taps:
            # [taps, channels]: a tap's weights of neighbouring channels lie side by side, as the kernel reads them
            self.conv_taps = torch.cat([tensors[n[k + "_conv"]] for k in kinds], dim=0).t().contiguous()
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
        if self.taps > 1:  # the convolution's last taps - 1 inputs, [taps - 1, channels]
            return StateNeed(((self.taps - 1) * self.channels,), torch.float32)
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
        if self.per_head:
            return self._forward_per_head(x, ctx, lane, writes)
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
                          self.keep_first, self.v_dim, self.wide_weights, self.chunk, self.softcap, sink=self.sink)
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
                      wide_weights=self.wide_weights, chunk=self.chunk, softcap=self.softcap, sink=self.sink)
        return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden), sink=sink)

    def _forward_per_head(self, x, ctx: StepContext, lane: LaneView, writes: bool):
        """Projection, the per-head steps and the attention (`forward_projected`), output projection."""
        proj = ops.linear(x, self.w_qkv, ctx.buffer("qkv_in" if self.taps > 1 else "qkv", self.w_qkv.shape[0]))
        attn = ctx.buffer("attn_out", self.o_in)
        self.forward_projected(proj, ctx, lane, writes, attn)
        return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden))

    # ---- optional: an arrangement that runs this mixer's projections inside larger products of its own ---------------------
    # (`packs_projections`: the mixer offers `input_weight` [columns, hidden] and `output_weight` [hidden, heads * v_dim], takes views
    # of the arrangement's packed matrices in their place (`adopt`), and runs everything between the two products on rows that the
    # arrangement hands it: `forward_projected`)
    @property
    def packs_projections(self) -> bool:
        return self.per_head

    @property
    def input_weight(self) -> torch.Tensor:
        return self.w_qkv

    @property
    def output_weight(self) -> torch.Tensor:
        return self.w_o

    def adopt(self, w_in: torch.Tensor, w_out: torch.Tensor) -> None:
        if w_in.shape != self.w_qkv.shape or w_out.shape != self.w_o.shape:
            raise ValueError("adopt: views of the projections' own shapes are needed")
        self.w_qkv, self.w_o = w_in, w_out

    def forward_projected(self, proj: torch.Tensor, ctx: StepContext, lane: LaneView, writes: bool, attn: torch.Tensor) -> None:
        """`proj` [N, >= columns of the packed projection] (rows may lie in a wider buffer): `ops.head_prepare_store` (convolution,
        head norms, rotation, query temperature, cache write), then attention with the sink and the heads' gates in its epilogue into
        `attn` [N, heads * v_dim] (likewise)."""
        if self.taps > 1 and not writes:
            raise ValueError("an attention mixer with a convolution owns its state: its lane cannot be shared")
        # a convolution reads its neighbours' rows: not in place
        qkv = ctx.buffer("qkv", self.w_qkv.shape[0]) if self.taps > 1 else proj
        pos, hn = self.position, self.head_norm
        rotates = pos is not None and pos.dims > 0
        ops.head_prepare_store(
            proj, qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim, self.v_dim,
            inv_freq=pos.inv_freq if rotates else None, magnitude=pos.magnitude if rotates else 1.0,
            interleaved=pos.interleaved if rotates else False, norm=hn.get("when", "before") if hn else None,
            q_gain=self.q_gain, k_gain=self.k_gain, eps=float(hn["eps"]) if hn else 0.0,
            q_temp=(float(self.q_temp["coef"]), float(self.q_temp["every"])) if self.q_temp else None,
            taps=self.conv_taps, v_from_k=self.v_from_k, write_kv=writes)
        gate = proj[:, self.channels: self.channels + self.heads] if self.head_gate else None
        ops.attention(qkv, lane, ctx, attn, self.heads, self.kv_heads, self.head_dim, self.scale, self.window, self.keep_first,
                      self.v_dim, self.wide_weights, self.chunk, self.softcap, sink=self.sink, gate=gate)
