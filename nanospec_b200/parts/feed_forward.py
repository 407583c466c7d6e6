"""The dense gated feed-forward of the reference (`MLP`, model/llama.py:187-195):
down(silu(gate(x)) * up(x)), no biases.  Gate and up are one packed projection: runs of 64 gate rows
followed by the 64 matching up rows when the intermediate size is a multiple of 64 (a decode step's
product then applies the activation in its epilogue), [gate | up] otherwise.

Interface of a feed-forward part:
    forward(x, ctx) -> y        x, y: [N, hidden] in the compute dtype
and, optionally, the folding of norms into its products (`Part.takes_row_scaled`, `Part.feeds_norm_sink`).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """params: hidden, intermediate, names (optional: the tensors' names after the part's prefix, keys "gate", "up",
    "down"; default the Hugging Face ones)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden"])
        self.inter = int(spec["intermediate"])
        names = dict(spec.params.get("names") or {})
        self.n_gate = names.get("gate", "gate_proj.weight")
        self.n_up = names.get("up", "up_proj.weight")
        self.n_down = names.get("down", "down_proj.weight")
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None
        self.gate_block = 0

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {
            self.n_gate: WeightSpec((self.inter, self.hidden)),
            self.n_up: WeightSpec((self.inter, self.hidden)),
            self.n_down: WeightSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        gate, up = tensors[self.n_gate], tensors[self.n_up]
        self.gate_block = ops.GATE_BLOCK if self.inter % ops.GATE_BLOCK == 0 else 0
        if self.gate_block:
            b = self.gate_block
            packed = torch.stack([gate.view(self.inter // b, b, self.hidden), up.view(self.inter // b, b, self.hidden)], dim=1)
            self.w_gate_up = packed.reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[self.n_down].contiguous()

    def takes_row_scaled(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_gate_up)

    def feeds_norm_sink(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_down)

    def forward(self, x, ctx: StepContext, sink: ops.NormSink | None = None):
        act = ops.gated_linear(x, self.w_gate_up, ctx.buffer("ffn_act", self.inter), ctx.buffer("gate_up", 2 * self.inter),
                               self.gate_block)
        return ops.linear(act, self.w_down, ctx.buffer("branch", self.hidden), sink=sink)


@register_part("feed_forward", "dense_act")
class DenseAct(Part):
    """down(act(up(x))), no gate, no biases.  params: hidden, intermediate, activation ("gelu_erf": the exact gelu,
    "gelu_tanh", "silu", "relu2": the square of relu), names (optional: keys "up", "down"; default "up", "down").  The activation is float32 on the
    rounded product and is rounded once.  `forward` takes `out_name`, the step buffer that receives the result (an arrangement that
    holds two branches at once gives another name than the mixers' "branch")."""

    names_output = True

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.hidden, self.inter = int(spec["hidden"]), int(spec["intermediate"])
        self.activation = spec.params.get("activation", "gelu_erf")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense_act: unknown activation {self.activation!r} (known: {', '.join(ops.ACTIVATIONS)})")
        names = dict(spec.params.get("names") or {})
        self.n_up, self.n_down = names.get("up", "up"), names.get("down", "down")
        self.w_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {self.n_up: WeightSpec((self.inter, self.hidden)), self.n_down: WeightSpec((self.hidden, self.inter))}

    def bind(self, tensors) -> None:
        self.w_up, self.w_down = tensors[self.n_up].contiguous(), tensors[self.n_down].contiguous()

    def forward(self, x, ctx: StepContext, out_name: str = "branch"):
        u = ops.linear(x, self.w_up, ctx.buffer("ffn_up", self.inter))
        a = ops.activation(u, ctx.buffer("ffn_act", self.inter), self.activation)
        return ops.linear(a, self.w_down, ctx.buffer(out_name, self.hidden))

    # ---- optional: an arrangement that runs the two products inside larger ones of its own (see `GQAAttention.packs_projections`)
    packs_projections = True

    @property
    def input_weight(self) -> torch.Tensor:
        return self.w_up

    @property
    def output_weight(self) -> torch.Tensor:
        return self.w_down

    def adopt(self, w_in: torch.Tensor, w_out: torch.Tensor) -> None:
        if w_in.shape != self.w_up.shape or w_out.shape != self.w_down.shape:
            raise ValueError("adopt: views of the projections' own shapes are needed")
        self.w_up, self.w_down = w_in, w_out

    def forward_projected(self, u: torch.Tensor, ctx: StepContext, act: torch.Tensor) -> None:
        """`u` [N, intermediate] (rows may lie in a wider buffer): the activation into `act` (likewise)."""
        ops.activation(u, act, self.activation)
