"""Norms over the float32 residual stream, fused with the residual sum: RMSNorm and a layer norm without bias.

Formula of the reference (model/llama.py:86-95): h = x * rsqrt(mean(x^2) + eps), y = gain * h,
eps inside the root, the gain applied as is (not 1 + gain).  Here the statistics, the scale
and the gain product are all float32 and the result is rounded once to the compute dtype.

Interface of a norm part:
    add_norm(resid, pending, ctx, rows=None, out_name="normed") -> normed
        resid    [N, H] float32, updated in place with `pending` when that is given
        pending  [N, H] compute dtype or None: a branch output not yet added to the stream
        rows     int32 device tensor or None: only these rows are produced (resid untouched)
        out_name the step buffer (`ctx.buffer(out_name, H, rows=...)`) that takes the result
    sink(resid, ctx) -> ops.NormSink    (optional) what a product needs to fold this norm and the sum
                                        before it into its epilogue; `add_norm` hands the product's
                                        `ops.RowScaled` result on unchanged.  A norm without `sink`
                                        is never folded.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: hidden, eps, weight_name (the gain's name after the norm's prefix; default "weight")."""

    centered = False
    bias: torch.Tensor | None = None

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden"])
        self.eps = float(spec["eps"])
        self.weight_name = spec.params.get("weight_name", "weight")
        self.gain: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden,), rule="float32", init="gain")}

    def bind(self, tensors) -> None:
        self.gain = tensors[self.weight_name].contiguous()

    def sink(self, resid: torch.Tensor, ctx: StepContext) -> ops.NormSink:
        return ops.NormSink(resid, self.gain, self.eps, ctx.workspace)

    def add_norm(self, resid: torch.Tensor, pending, ctx: StepContext,
                 rows: torch.Tensor | None = None, out_name: str = "normed"):
        if isinstance(pending, ops.RowScaled):
            # a product has added its output to the stream and prepared this norm's input already
            if pending.gain is not self.gain or rows is not None:
                raise ValueError("a RowScaled reached a norm it was not made for")
            return pending
        n = resid.shape[0] if rows is None else rows.numel()
        out = ctx.buffer(out_name, self.hidden, rows=n)
        return ops.add_rmsnorm(resid, pending, self.gain, self.eps, out, rows=rows)


@register_part("norm", "layernorm")
class LayerNorm(RMSNorm):
    """(x - mean) / sqrt(var + eps) * gain (+ bias): the variance is the mean of the squared deviations.
    Mean and variance are taken in float32 in two passes over the row.  It has no `sink`: a centred norm is not a
    per-row scale of the stream, so it is never folded into the products around it.  params as `rmsnorm`, and
    bias_name (the bias's name after the norm's prefix; default None: no bias)."""

    sink = None  # hasattr(norm, "sink") is what the blocks ask; None says it cannot be folded
    centered = True

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.bias_name = spec.params.get("bias_name")
        self.bias: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        specs = super().weight_specs()
        if self.bias_name is not None:
            specs[self.bias_name] = WeightSpec((self.hidden,), rule="float32", init="normal")
        return specs

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.bias_name is not None:
            self.bias = tensors[self.bias_name].contiguous()

    def add_norm(self, resid: torch.Tensor, pending, ctx: StepContext,
                 rows: torch.Tensor | None = None, out_name: str = "normed"):
        if isinstance(pending, ops.RowScaled):
            raise ValueError("a RowScaled reached a norm that cannot take it")
        n = resid.shape[0] if rows is None else rows.numel()
        out = ctx.buffer(out_name, self.hidden, rows=n)
        if self.bias is not None:  # the kernel of the streams, on one stream: the residual sum, the norm and its bias
            return ops.stream_mix_norm(resid, 1, pending, None, None, None, self.gain, self.bias, self.eps, True, out, rows=rows)
        return ops.add_layernorm(resid, pending, self.gain, self.eps, out, rows=rows)


@register_part("norm", "dyt")
class DynamicTanh(Part):
    """tanh(alpha * x) * gain + bias: a norm that takes no mean and no variance (one scalar `alpha` stored beside the gain and
    the bias), elementwise in float32 over the float32 stream and rounded once.  It is not a per-row scale, so it offers no `sink`
    (the folding of RMS norms); being elementwise, it offers `elementwise_sink` instead: a product of up to 64 tokens whose output
    joins the stream right before this norm applies it in its epilogue.  `add_norm` also takes a tuple of two pending branches (what a block that
    runs its sublayers side by side leaves).  params: hidden, weight_name (default "weight"), bias_name (default weight_name +
    ".b"), alpha_name (default weight_name + ".alpha"); names follow the norm's prefix directly."""

    sink = None
    centered = False
    takes_branches = 2  # `add_norm` accepts a tuple of so many pending branches

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden"])
        self.weight_name = spec.params.get("weight_name", "weight")
        self.bias_name = spec.params.get("bias_name", self.weight_name + ".b")
        self.alpha_name = spec.params.get("alpha_name", self.weight_name + ".alpha")
        self.gain: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.alpha: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden,), rule="float32", init="gain"),
                self.bias_name: WeightSpec((self.hidden,), rule="float32", init="normal", std=0.1),
                self.alpha_name: WeightSpec((), rule="float32", init="gain")}

    def bind(self, tensors) -> None:
        self.gain = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.bias_name].contiguous()
        self.alpha = tensors[self.alpha_name].reshape(1).contiguous()

    def elementwise_sink(self, resid: torch.Tensor, ctx: StepContext) -> ops.TanhSink:
        """What a product needs to fold this norm and the residual sum before it into its epilogue (`ops.linear(..., sink=)`): the
        norm is elementwise, so the product's epilogue leaves its result complete (`ops.Normed`), which `add_norm` hands on."""
        return ops.TanhSink(resid, self.gain, self.bias, self.alpha, ctx.workspace)

    def add_norm(self, resid: torch.Tensor, pending, ctx: StepContext,
                 rows: torch.Tensor | None = None, out_name: str = "normed"):
        if isinstance(pending, ops.RowScaled):
            raise ValueError("a RowScaled reached a norm that cannot take it")
        if isinstance(pending, ops.Normed):
            # a product has added its output to the stream and applied this norm already
            if pending.gain is not self.gain or rows is not None:
                raise ValueError("a Normed reached a norm it was not made for")
            return pending.x
        branches = pending if isinstance(pending, (tuple, list)) else (pending,)
        n = resid.shape[0] if rows is None else rows.numel()
        out = ctx.buffer(out_name, self.hidden, rows=n)
        return ops.add_dyt(resid, branches, self.gain, self.bias, self.alpha, out, rows=rows)
