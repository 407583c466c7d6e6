"""Token embedding into the float32 residual stream (model/llama.py:214,221: a plain row
gather, no scaling) and the output head (model/llama.py:262,286: logits = h W^T, no bias, no
soft-cap), which may share the embedding's table."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("embedding", "table")
class TokenEmbedding(Part):
    """params: vocab, hidden, weight_name (the table's name after the part's prefix; default "weight"), scale (the rows
    are multiplied by it; default 1) and copies (the stream is opened as so many equal copies side by side in a row,
    for a block arrangement that keeps several; default 1).  side_name and side_columns (optional): a second table
    [vocab, side_columns] under that name, whose row of a token the layers read slices of (`ctx.extras["token_side"]`
    is the table; a layer indexes it with the step's token ids on the device, so nothing is gathered here)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.weight_name = spec.params.get("weight_name", "weight")
        self.scale = float(spec.params.get("scale") or 1.0)
        self.copies = int(spec.params.get("copies") or 1)
        self.side_name = spec.params.get("side_name")
        self.side_columns = int(spec.params.get("side_columns") or 0)
        self.table: torch.Tensor | None = None
        self.side_table: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        specs = {self.weight_name: WeightSpec((self.vocab, self.hidden))}
        if self.side_name:
            specs[self.side_name] = WeightSpec((self.vocab, self.side_columns), std=1.0)
        return specs

    def bind(self, tensors) -> None:
        self.table = tensors[self.weight_name].contiguous()
        if self.side_name:
            self.side_table = tensors[self.side_name].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        if self.side_table is not None:
            ctx.extras["token_side"] = self.side_table
        if self.scale != 1.0 or self.copies != 1:
            return ops.embed_streams(self.table, ctx.token_ids, ctx.buffer("resid", self.copies * self.hidden, torch.float32),
                                     self.scale, self.copies)
        return ops.embed(self.table, ctx.token_ids, ctx.buffer("resid", self.hidden, torch.float32))


@register_part("head", "linear")
class LinearHead(Part):
    """params: vocab, hidden, tied_to (full name of the embedding table, or None), weight_name (default "weight"),
    scale (the logits are multiplied by it; default 1) and softcap (c > 0: logits = c * tanh(logits / c), after the
    scale; default none)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.tied_to = spec.params.get("tied_to")
        self.weight_name = spec.params.get("weight_name", "weight")
        self.scale = float(spec.params.get("scale") or 1.0)
        self.softcap = float(spec.params.get("softcap") or 0.0)
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab, self.hidden), alias=self.tied_to)}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.weight_name]

    def forward(self, h: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """h [R, hidden] compute dtype -> float32 logits [R, vocab]."""
        if out is None:
            out = torch.empty((h.shape[0], self.vocab), dtype=torch.float32, device=h.device)
        ops.linear(h, self.weight, out)
        if self.scale != 1.0 or self.softcap > 0.0:
            ops.scale_softcap(out, self.scale, self.softcap)
        return out
