"""Typed configuration of the Debuvik decoder, read from its own config.json.

A Debuvik model is a list of layers that norm what a sublayer returns (x = x + norm(sublayer(x)), an RMS norm; the
sublayers read the stream itself).  A layer's mixer is attention over a cached latent without positions, with a sigmoid
gate on every output feature, or grouped-query attention with biases, an RMS norm over the whole q and the whole k
projection, a rotation of the leading features of each head, capped scores and a mask of chunks - optionally on the keys and
values that an earlier layer stored.  A gated feed-forward follows (or none), and then, when the model has a second
embedding table, the layer's own slice of the token's row of it, gated by the stream.  Every size and every constant that
can differ between models comes from the file:

    architecture "Debuvik";  vocab, width;  norm.eps;  token_side {dim} (optional)
    layers[i]: type ("latent_attention" | "attention"), mixer {...}, mlp {kind "dense", ff} or null
      latent_attention: heads, dim, vdim, kv_rank, scale
      attention:        heads, kv_heads, dim, vdim, scale, softcap (optional), mask {size} (optional), kv_from (optional),
                        rot {dims, base, scaling {factor, low, high, original} (optional)} (optional)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .files import ConfigError

MIXER_TYPES = ("latent_attention", "attention")
MAX_POSITIONS = 1 << 20  # the file gives no limit; positions are 32-bit and angles float32


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Debuvik config: {where} lacks {key!r}")
    return d[key]


@dataclass(frozen=True)
class DebuvikLayer:
    type: str
    mixer: dict[str, Any]
    ff: int | None  # None: no feed-forward

    @property
    def kv_from(self) -> int | None:
        v = self.mixer.get("kv_from")
        return None if v is None else int(v)

    def to_hf(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer, "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class DebuvikConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[DebuvikLayer, ...]
    side_dim: int = 0  # columns of the second embedding table that each layer reads; 0: the model has none
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Debuvik"

    @classmethod
    def from_hf(cls, cfg: dict[str, Any], generation: dict[str, Any] | None = None) -> "DebuvikConfig":
        if cfg.get("architecture") != "Debuvik" and "Debuvik" not in (cfg.get("architectures") or []):
            raise ConfigError(f"not a Debuvik config: architecture={cfg.get('architecture')!r}")
        entries = _need(cfg, "layers", "config.json")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"Debuvik config: {where} has the unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = dict(_need(entry, "mixer", where))
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank", "scale"):
                    _need(m, key, where + ".mixer")
            else:
                for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                    _need(m, key, where + ".mixer")
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"Debuvik config: {where}: {m['heads']} query heads over {m['kv_heads']} key/value heads")
                if m.get("mask") is not None:
                    m["mask"] = {"size": int(_need(m["mask"], "size", where + ".mixer.mask"))}
                    if m["mask"]["size"] < 1:
                        raise ConfigError(f"Debuvik config: {where}: chunks of {m['mask']['size']} positions")
                if m.get("rot") is not None:
                    rot = dict(m["rot"])
                    for key in ("dims", "base"):
                        _need(rot, key, where + ".mixer.rot")
                    if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"]):
                        raise ConfigError(f"Debuvik config: {where}: {rot['dims']} of {m['dim']} features cannot turn in pairs")
                    if rot.get("scaling"):
                        for key in ("factor", "low", "high", "original"):
                            _need(rot["scaling"], key, where + ".mixer.rot.scaling")
                    m["rot"] = rot
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or entries[src].get("type") != "attention" or (entries[src].get("mixer") or {}).get("kv_from") is not None:
                        raise ConfigError(f"Debuvik config: {where} takes keys and values from layer {src}, which is no earlier "
                                          "attention layer with projections of its own")
                    sm = entries[src]["mixer"]
                    if any(int(sm[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"Debuvik config: {where} and layer {src}, whose keys and values it reads, differ in size")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"Debuvik config: {where} has the unknown feed-forward kind {mlp.get('kind')!r}")
                ff = int(_need(mlp, "ff", where + ".mlp"))
            layers.append(DebuvikLayer(kind, m, ff))
        side = cfg.get("token_side")
        side_dim = int(_need(side, "dim", "token_side")) if side is not None else 0
        eos = (generation or {}).get("eos_token_id", cfg.get("eos_token_id"))
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=int(_need(cfg, "vocab", "config.json")), width=int(_need(cfg, "width", "config.json")),
                   eps=float(_need(_need(cfg, "norm", "config.json"), "eps", "norm")), layers=tuple(layers),
                   side_dim=side_dim, eos_token_ids=eos_ids)

    def to_hf(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps}, "layers": [layer.to_hf() for layer in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
