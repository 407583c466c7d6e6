"""How a layer's parts are arranged.  "prenorm" is the reference's `DecoderLayer`
(model/llama.py:198-208): x = x + mixer(norm(x)); x = x + feed_forward(norm(x)).

A block receives the float32 residual stream and a `pending` branch output that has not
been added to it yet, and returns the same pair; the sum is folded into the next norm so
that each activation is read once.

In a decode step of a few tokens the two norm kernels of a layer can go: when the part before a
norm can feed a sink and the part after it takes row-scaled input (`Part.feeds_norm_sink`,
`Part.takes_row_scaled`), the product before the norm adds its output to the stream and prepares the
norm's input in its epilogue, and the product after it applies the norm's scale.  `follow` is the
block that runs next (or None): its first norm is the one after this block's feed-forward.

Interface of a block part (built from a whole `LayerSpec`):
    mixer                                          the block's mixer part: the model asks it for the lane's cache and state needs
    parts() -> dict of slot name -> Part           (for weight naming: `LayerSpec.names` maps each slot to its sub-prefix)
    forward(resid, pending, ctx, lane, writes) -> (resid, pending)
    takes_follow = True                            (optional) forward() also accepts `follow=`, the block that runs next
    input_norm_sink(resid, ctx) -> ops.NormSink or None   (optional; None or absent: the block's first norm cannot be folded)
The built-in mixers and feed-forwards return their result in the step's "branch" buffer: an arrangement that needs
two branch outputs at once copies the first before it runs the second.

"outnorm" norms what a sublayer returns instead of what it reads: x = x + norm(mixer(x)); x = x + norm(feed_forward(x)),
then, when the layer has one, x = x + norm(side_input(x)) (`LayerSpec.params["side_input"]`, a `PartSpec` of the
"side_input" slot; checkpoint sub-prefix under the slot name "side_input").  The sublayers read the stream itself, so
nothing stays pending: one kernel (`ops.norm_add`) norms the branch, adds it to the float32 stream and leaves the
stream's copy in the compute type for the next sublayer; the block hands that copy on as a `StreamCopy`.

"parallel" has one norm and both sublayers read its output: h = norm(x); x = x + (mixer(h) + feed_forward(h)).  Neither branch is
added by a kernel of its own when the norm that comes next takes two pending branches (`takes_branches`, as the "dyt" norm does):
the block leaves the pair pending and that norm's kernel sums stream, mixer branch and feed-forward branch in float32.  Otherwise the
mixer's branch joins the stream through `ops.residual_add` and the feed-forward's stays pending as a tensor.
When both sublayers offer their projections (`packs_projections`) the block runs TWO products a layer instead of four: one packed
input projection [mixer's columns | feed-forward's] of h, and one output projection of the concatenated [heads' outputs |
activations] by [W_o | W_down], whose float32 accumulator holds mixer(h) + feed_forward(h) before it is rounded once; the sublayers
keep views of the packed matrices in place of their own (`adopt`), so weights are held once and replaced in place.  In a step of up
to 64 tokens the packed output product also adds its result to the stream and applies the NEXT block's norm in its epilogue, when
that norm is elementwise (`elementwise_sink`): a decode layer is then five kernels and the tail of a convolution.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..config.recipe import LayerSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


def _folds(norm) -> bool:
    """Whether a norm can be folded into the products around it (it offers `sink`)."""
    return callable(getattr(norm, "sink", None))


def _can(part, what: str, n_tokens: int) -> bool:
    """A part's optional capability (`takes_row_scaled`, `feeds_norm_sink`); parts that do not know of it have none."""
    f = getattr(part, what, None)
    return bool(f(n_tokens)) if callable(f) else False


@register_part("block", "prenorm")
class PreNormBlock:
    slots = ("norm_mixer", "mixer", "norm_feed_forward", "feed_forward")
    takes_follow = True  # forward() accepts the block that runs next

    def __init__(self, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.layer = layer
        self.mixer = build_part("mixer", layer.mixer, dtype, device)
        self.norm_mixer = build_part("norm", layer.norm, dtype, device)
        # a layer without a feed-forward (`LayerSpec.feed_forward` None) is its first sublayer alone
        self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device) if layer.feed_forward is not None else None
        self.norm_feed_forward = build_part("norm", layer.norm, dtype, device) if layer.feed_forward is not None else None

    def parts(self) -> dict:
        return {s: getattr(self, s) for s in self.slots if getattr(self, s) is not None}

    def input_norm_sink(self, resid: torch.Tensor, ctx: StepContext):
        """What the product before this block needs to fold the block's first norm in, or None."""
        if _can(self.mixer, "takes_row_scaled", ctx.n_tokens) and _folds(self.norm_mixer):
            return self.norm_mixer.sink(resid, ctx)
        return None

    def forward(self, resid: torch.Tensor, pending, ctx: StepContext, lane: LaneView, writes: bool = True,
                follow=None) -> tuple[torch.Tensor, torch.Tensor]:
        n = ctx.n_tokens
        x = self.norm_mixer.add_norm(resid, pending, ctx)
        if self.feed_forward is None:
            sink = None
            if follow is not None and _can(self.mixer, "feeds_norm_sink", n) and hasattr(follow, "input_norm_sink"):
                sink = follow.input_norm_sink(resid, ctx)
            if sink is not None:
                return resid, self.mixer.forward(x, ctx, lane, writes, sink=sink)
            return resid, self.mixer.forward(x, ctx, lane, writes)
        if _can(self.mixer, "feeds_norm_sink", n) and _can(self.feed_forward, "takes_row_scaled", n) \
                and _folds(self.norm_feed_forward):
            a = self.mixer.forward(x, ctx, lane, writes, sink=self.norm_feed_forward.sink(resid, ctx))
        else:
            a = self.mixer.forward(x, ctx, lane, writes)
        x = self.norm_feed_forward.add_norm(resid, a, ctx)
        sink = None
        if follow is not None and _can(self.feed_forward, "feeds_norm_sink", n) and hasattr(follow, "input_norm_sink"):
            sink = follow.input_norm_sink(resid, ctx)
        if sink is not None:
            return resid, self.feed_forward.forward(x, ctx, sink=sink)
        return resid, self.feed_forward.forward(x, ctx)


@dataclass
class StreamCopy:
    """What an "outnorm" block hands its successor in place of a pending branch: nothing is pending, and `x` is the
    stream as it stands, in the compute type (in float32 the stream itself)."""

    x: torch.Tensor


@register_part("block", "outnorm")
class OutNormBlock:
    slots = ("mixer", "norm_mixer", "feed_forward", "norm_feed_forward", "side_input")

    def __init__(self, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.layer = layer
        self.dtype = dtype
        self.mixer = build_part("mixer", layer.mixer, dtype, device)
        self.norm_mixer = build_part("norm", layer.norm, dtype, device)
        has_ff = layer.feed_forward is not None
        self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device) if has_ff else None
        self.norm_feed_forward = build_part("norm", layer.norm, dtype, device) if has_ff else None
        side = layer.params.get("side_input")
        self.side_input = build_part("side_input", side, dtype, device) if side is not None else None
        for norm in (self.norm_mixer, self.norm_feed_forward):
            if norm is not None and (not hasattr(norm, "gain") or getattr(norm, "centered", False) or getattr(norm, "bias", None) is not None):
                raise ValueError("the outnorm arrangement folds its norms into the residual sum: an RMS norm part with `gain` and `eps` is needed")

    def parts(self) -> dict:
        return {s: getattr(self, s) for s in self.slots if getattr(self, s) is not None}

    def _copy(self, resid: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if self.dtype == torch.float32:
            return resid
        return ctx.buffer("stream_copy", resid.shape[1])

    def _join(self, resid: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float, ctx: StepContext,
              bias: torch.Tensor | None = None) -> torch.Tensor:
        """resid += norm(y + bias) * gain; returns the stream's copy in the compute type."""
        x = self._copy(resid, ctx)
        ops.norm_add(resid, y, gain, eps, cast=None if x is resid else x, bias=bias)
        return x

    def forward(self, resid: torch.Tensor, pending, ctx: StepContext, lane: LaneView, writes: bool = True):
        if isinstance(pending, StreamCopy):
            x = pending.x
        else:
            if pending is not None:  # a block of another kind ran before: its branch joins the stream as it is
                if not isinstance(pending, torch.Tensor):
                    raise ValueError("the outnorm arrangement follows a block that leaves a tensor, or one of its own kind")
                ops.residual_add(resid, pending)
            x = self._copy(resid, ctx)
            if x is not resid:
                ops.norm_add(resid, None, None, 0.0, cast=x)
        # a mixer that ends in a bias (`branch_bias`) leaves it to the norm's kernel, which adds it before the statistics
        bias = getattr(self.mixer, "branch_bias", None)
        y = self.mixer.forward(x, ctx, lane, writes, leave_bias=True) if bias is not None else self.mixer.forward(x, ctx, lane, writes)
        x = self._join(resid, y, self.norm_mixer.gain, self.norm_mixer.eps, ctx, bias)
        if self.feed_forward is not None:
            x = self._join(resid, self.feed_forward.forward(x, ctx), self.norm_feed_forward.gain, self.norm_feed_forward.eps, ctx)
        if self.side_input is not None:
            x = self._join(resid, self.side_input.forward(x, ctx), self.side_input.gain, self.side_input.eps, ctx)
        return resid, StreamCopy(x)

    def close(self, resid: torch.Tensor, pending, norm, ctx: StepContext, rows: torch.Tensor | None = None,
              out_name: str = "final_normed") -> torch.Tensor:
        """The model's end: nothing is pending, the final norm reads the stream; only `rows` when given."""
        return norm.add_norm(resid, None, ctx, rows=rows, out_name=out_name)


@register_part("block", "parallel")
class ParallelBlock:
    slots = ("norm_mixer", "mixer", "feed_forward")
    takes_follow = True
    PACK = True  # False: the sublayers run their own products (measurements and tests of that path)

    def __init__(self, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.layer = layer
        self.mixer = build_part("mixer", layer.mixer, dtype, device)
        self.norm_mixer = build_part("norm", layer.norm, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device) if layer.feed_forward is not None else None
        self.w_in: torch.Tensor | None = None   # [mixer's columns + feed-forward's, hidden] once packed
        self.w_out: torch.Tensor | None = None  # [hidden, heads' outputs + activations]
        self._packed: bool | None = None        # decided when the weights are bound

    def parts(self) -> dict:
        return {s: getattr(self, s) for s in self.slots if getattr(self, s) is not None}

    def takes_pair(self) -> bool:
        """Whether this block's norm sums two pending branches into the stream itself."""
        return int(getattr(self.norm_mixer, "takes_branches", 1)) >= 2

    @staticmethod
    def _settle(resid: torch.Tensor, pending):
        """A pending pair as one pending tensor: the first branch joins the stream now."""
        if isinstance(pending, tuple):
            ops.residual_add(resid, pending[0])
            return pending[1]
        return pending

    def _pack(self) -> bool:
        """Packs the sublayers' projections once.  Widths in multiples of eight only: rows of the packed buffers then start on 16 bytes
        in bfloat16, which the sublayers' kernels ask of their operands."""
        m, f = self.mixer, self.feed_forward
        if not (self.PACK and f is not None and getattr(m, "packs_projections", False) and getattr(f, "packs_projections", False)):
            return False
        wi_m, wi_f, wo_m, wo_f = m.input_weight, f.input_weight, m.output_weight, f.output_weight
        if any(w is None for w in (wi_m, wi_f, wo_m, wo_f)) or any(w.shape[0] % 8 or w.shape[1] % 8 for w in (wi_m, wi_f, wo_m, wo_f)):
            return False
        self.w_in = torch.cat([wi_m, wi_f], dim=0).contiguous()
        self.w_out = torch.cat([wo_m, wo_f], dim=1).contiguous()
        m.adopt(self.w_in[: wi_m.shape[0]], self.w_out[:, : wo_m.shape[1]])
        f.adopt(self.w_in[wi_m.shape[0]:], self.w_out[:, wo_m.shape[1]:])
        return True

    def after_bind(self) -> None:
        """Called by the model once every part has its weights."""
        self._packed = self._pack()

    def forward(self, resid: torch.Tensor, pending, ctx: StepContext, lane: LaneView, writes: bool = True, follow=None):
        if self._packed is None:  # parts bound by hand: pack now, unless a graph is being captured (no allocation then)
            self._packed = False if torch.cuda.is_current_stream_capturing() else self._pack()
        if isinstance(pending, tuple) and not self.takes_pair():
            pending = self._settle(resid, pending)
        h = self.norm_mixer.add_norm(resid, pending, ctx)
        if self._packed:
            cm, om = self.mixer.input_weight.shape[0], self.mixer.output_weight.shape[1]
            proj = ops.linear(h, self.w_in, ctx.buffer("par_in", self.w_in.shape[0]))
            mid = ctx.buffer("par_mid", self.w_out.shape[1])
            self.mixer.forward_projected(proj[:, :cm], ctx, lane, writes, mid[:, :om])
            self.feed_forward.forward_projected(proj[:, cm:], ctx, mid[:, om:])
            # a step of a few tokens: the sum into the stream and the next block's norm in this product's epilogue
            sink = None
            nxt = getattr(follow, "norm_mixer", None) if isinstance(follow, ParallelBlock) else None
            if nxt is not None and callable(getattr(nxt, "elementwise_sink", None)) and ops.norm_fusion_ok(ctx.n_tokens, self.w_out.dtype, self.w_out):
                sink = nxt.elementwise_sink(resid, ctx)
            return resid, ops.linear(mid, self.w_out, ctx.buffer("branch", resid.shape[1]), sink=sink)
        a = self.mixer.forward(h, ctx, lane, writes)
        if self.feed_forward is None:
            return resid, a
        # the pair stays pending only for a norm that is known to take it: the next block's, when that is of this kind
        pair = getattr(self.feed_forward, "names_output", False) and isinstance(follow, ParallelBlock) and follow.takes_pair()
        if pair:
            return resid, (a, self.feed_forward.forward(h, ctx, out_name="branch_ff"))
        ops.residual_add(resid, a)
        return resid, self.feed_forward.forward(h, ctx)

    def close(self, resid: torch.Tensor, pending, norm, ctx: StepContext, rows: torch.Tensor | None = None,
              out_name: str = "final_normed") -> torch.Tensor:
        """The model's end: the final norm takes what is pending."""
        if isinstance(pending, tuple) and int(getattr(norm, "takes_branches", 1)) < 2:
            pending = self._settle(resid, pending)
        return norm.add_norm(resid, pending, ctx, rows=rows, out_name=out_name)
