"""A layer's own input from the token itself: a slice of a second embedding row of the token, gated by the stream.

    e = side_table[token][index * dim : (index + 1) * dim]
    g = gelu_tanh(W_gate x) * e                      W_gate [dim, hidden]
    y = W_proj g                                     W_proj [hidden, dim]

The arrangement that owns the part norms y with the part's `gain` (an RMS norm with a plain gain) as it adds it to the
stream.  The table belongs to the embedding (`side_name` of the "table" embedding, which leaves it in
`ctx.extras["token_side"]`); the kernel reads the token's row through the step's token ids on the device, so the part
runs under CUDA graphs.

params: hidden, dim, index (which slice of the table's row is this layer's), eps, names (optional: keys "gate", "proj",
"norm"; default those words).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("side_input", "token_gate")
class TokenGate(Part):
    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden, self.dim, self.index = int(p["hidden"]), int(p["dim"]), int(p["index"])
        self.eps = float(p["eps"])
        names = dict(p.get("names") or {})
        self.n_gate, self.n_proj, self.n_norm = names.get("gate", "gate"), names.get("proj", "proj"), names.get("norm", "norm")
        self.w_gate = self.w_proj = self.gain = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {self.n_gate: WeightSpec((self.dim, self.hidden)), self.n_proj: WeightSpec((self.hidden, self.dim)),
                self.n_norm: WeightSpec((self.hidden,), rule="float32", init="gain")}

    def bind(self, tensors) -> None:
        self.w_gate, self.w_proj = tensors[self.n_gate].contiguous(), tensors[self.n_proj].contiguous()
        self.gain = tensors[self.n_norm].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        table = ctx.extras.get("token_side")
        if table is None or table.shape[1] < (self.index + 1) * self.dim:
            raise ValueError("a token_gate part needs an embedding with a side table of at least (index + 1) * dim columns")
        a = ops.linear(x, self.w_gate, ctx.buffer("side_gate", self.dim))
        g = ops.token_gate(a, table, ctx.token_ids, self.index * self.dim, ctx.buffer("side_act", self.dim))
        return ops.linear(g, self.w_proj, ctx.buffer("branch", self.hidden))
