"""Rotary position encoding, with the llama3 wavelength-banded frequency rescale.

The frequencies are computed once, in float32, with the reference's expressions in the
reference's order (model/llama.py:98-118); the kernel forms angle = float(position) *
inv_freq[j] in float32 and rotates the pairs (j, j + head_dim/2) ("rotate half",
model/llama.py:150-158).

Interface of a position part used by an attention mixer:
    rotate_and_store(qkv, ctx, lane, nq, nkv, head_dim, writes)
        rotates q and k inside the packed projection [q | k | v]; when `writes`, stores the
        rotated k and v at each token's slot of `lane`.
    project_rotate_store(x, w_qkv, qkv, ctx, lane, nq, nkv, head_dim, writes) -> bool      (optional)
        the projection itself with the rotation and the store in its epilogue; False (nothing done)
        when the step does not fit, and the mixer then runs the projection and `rotate_and_store`.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import Part
from .context import LaneView, StepContext
from .registry import register_part


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """float32 [head_dim / 2] on the CPU; `scaling` holds the llama3 block or is None."""
    ar = torch.arange(0, head_dim, 2, dtype=torch.int64).float()
    inv_freq = 1.0 / (theta ** (ar / head_dim))
    if scaling is None:
        return inv_freq
    factor = scaling["factor"]
    low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
    old_len = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = old_len / low, old_len / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_len / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) * ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled)


@register_part("position", "rope")
class RotaryEncoding(Part):
    """params: head_dim, theta, scaling (None or the llama3 block as a dict)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.head_dim = int(spec["head_dim"])
        scaling = spec.params.get("scaling")
        self.inv_freq_host = rope_inverse_frequencies(self.head_dim, float(spec["theta"]),
                                                      dict(scaling) if scaling else None)
        self._inv_freq: torch.Tensor | None = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            self._inv_freq = self.inv_freq_host.to(self.device).contiguous()
        return self._inv_freq

    def rotate_and_store(self, qkv: torch.Tensor, ctx: StepContext, lane: LaneView, nq: int, nkv: int,
                         head_dim: int, writes: bool) -> None:
        ops.rope_kv_write(qkv, ctx.positions, ctx.token_req, lane.block_table, self.inv_freq, lane.k, lane.v,
                          lane.page_size, nq, nkv, head_dim, write_kv=writes)

    def project_rotate_store(self, x, w_qkv: torch.Tensor, qkv: torch.Tensor, ctx: StepContext, lane: LaneView, nq: int,
                             nkv: int, head_dim: int, writes: bool) -> bool:
        return ops.linear_rope(x, w_qkv, qkv, ctx.positions, ctx.token_req, lane.block_table, self.inv_freq, lane.k, lane.v,
                               lane.page_size, nq, nkv, head_dim, write_kv=writes)


def rotary_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """Frequencies of the dims / 2 rotated pairs (float32 on the CPU) and the factor on cos and sin.

    Without scaling f_i = base^(-2i / dims).  With the YaRN block (`factor`, `original`, `fast`, `slow`): a pair
    that makes `t` turns over `original` positions sits at d(t) = dims * ln(original / (2 pi t)) / (2 ln base);
    pairs up to floor(d(fast)) keep f_i, pairs from ceil(d(slow)) on turn `factor` times slower, and a linear
    ramp joins them; cos and sin are multiplied by 0.1 * ln(factor) + 1.
    """
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f.to(torch.float32), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if "low" in scaling or "high" in scaling:
        # the wavelength bands (`factor`, `low`, `high`, `original`): with wavelength l = 2 pi / f, a pair with
        # l < original / high keeps f, one with l > original / low turns `factor` times slower, and between the two
        # s = (original / l - low) / (high - low) blends them, (1 - s) f / factor + s f; cos and sin are not scaled
        low, high = float(scaling["low"]), float(scaling["high"])
        wave = 2.0 * math.pi / f
        s = (original / wave - low) / (high - low)
        banded = torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, (1.0 - s) * f / factor + s * f))
        return banded.to(torch.float32), 1.0

    def at(turns: float) -> float:
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(float(base)))

    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


@register_part("position", "rotary")
class Rotary(Part):
    """Rotation of the first `dims` features of every q and k head, in either pairing.

    params: head_dim, dims (how many features turn, even, at most head_dim), base, layout ("half": pairs
    (i, i + dims/2); "interleaved": pairs (2i, 2i + 1)), scaling (None, the YaRN block {factor, original, fast, slow} or
    the wavelength bands {factor, original, low, high}, see `rotary_frequencies`).
    An attention mixer calls `rotate_and_store` (which can also norm the whole q and k projections first and takes
    values of another width than the keys); a mixer with a state reads `inv_freq`, `magnitude` and `interleaved`.
    """

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.head_dim = int(spec["head_dim"])
        self.dims = int(spec.params.get("dims", self.head_dim))
        layout = spec.params.get("layout", "half")
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rotary: unknown layout {layout!r}")
        if self.dims % 2 or not 0 <= self.dims <= self.head_dim:
            raise ValueError(f"rotary: {self.dims} of {self.head_dim} features cannot be rotated in pairs")
        self.interleaved = layout == "interleaved"
        scaling = spec.params.get("scaling")
        self.inv_freq_host, self.magnitude = rotary_frequencies(self.dims, float(spec["base"]), dict(scaling) if scaling else None)
        self._inv_freq: torch.Tensor | None = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            self._inv_freq = self.inv_freq_host.to(self.device).contiguous()
        return self._inv_freq

    def rotate_and_store(self, qkv: torch.Tensor, ctx: StepContext, lane: LaneView, nq: int, nkv: int, head_dim: int,
                         writes: bool, v_dim: int | None = None, q_gain=None, k_gain=None, eps: float = 0.0, bias=None) -> None:
        """`bias`: the projections' bias, one float32 per feature of the row, added before the norm.  `nkv` 0: the rows
        hold queries alone (the mixer reads keys and values that another layer stored)."""
        ops.qk_norm_rope_store(qkv, ctx, lane, self.inv_freq if self.dims else None, self.magnitude, self.interleaved, nq, nkv,
                               head_dim, head_dim if v_dim is None else v_dim, q_gain, k_gain, eps, write_kv=writes, bias=bias)
