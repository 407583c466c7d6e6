"""Typed configuration of the Fubolix decoder, read from its own config.json.

A Fubolix model is a list of layers with one norm each - a dynamic tanh, which takes no statistics - whose output both the
mixer and the feed-forward read: x = x + (mixer(h) + feed_forward(h)), h = norm(x).  The mixer is one of three kinds of
softmax attention, all with a sink in the denominator; the feed-forward is dense with a squared relu, or absent.  Every size
and every constant that can differ between models comes from the file:

    architecture "Fubolix";  vocab, width;  norm.eps;  embedding.scale
    layers[i]: type ("attention" | "attention_2" | "attention_3"), mixer {...}, mlp {kind "dense", ff} or null
      attention:   heads, kv_heads, dim, vdim, scale, mask {size, keep_first}, rot {dims, base, scaling {factor, original, fast, slow}}
      attention_2: heads, kv_heads, dim, vdim, scale, q_temp {coef, every}
      attention_3: heads, kv_heads, dim, vdim, scale, conv, rot {dims, base, scaling {...}}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .files import ConfigError

MIXER_TYPES = ("attention", "attention_2", "attention_3")
MAX_POSITIONS = 1 << 20  # the file gives no limit; positions are 32-bit and angles float32

_REQUIRED = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"),
    "attention_2": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "attention_3": ("heads", "kv_heads", "dim", "vdim", "scale", "conv", "rot"),
}


def _need(d: Any, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Fubolix config: {where} lacks {key!r}")
    return d[key]


def _rot(m: dict, where: str) -> dict:
    rot = dict(m["rot"])
    for key in ("dims", "base"):
        _need(rot, key, where + ".rot")
    rot["dims"], rot["base"] = int(rot["dims"]), float(rot["base"])
    if rot["dims"] % 2 or not 0 <= rot["dims"] <= int(m["dim"]):
        raise ConfigError(f"Fubolix config: {where}.rot turns {rot['dims']} of {m['dim']} features")
    sc = rot.get("scaling")
    if sc:
        for key in ("factor", "original", "fast", "slow"):
            _need(sc, key, where + ".rot.scaling")
        rot["scaling"] = {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")}
    else:
        rot["scaling"] = None
    return rot


@dataclass(frozen=True)
class FubolixLayer:
    type: str
    mixer: dict[str, Any]
    ff: int | None  # None: no feed-forward

    def to_hf(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer, "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class FubolixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[FubolixLayer, ...]
    embedding_scale: float = 1.0
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Fubolix"

    @classmethod
    def from_hf(cls, cfg: dict[str, Any], generation: dict[str, Any] | None = None) -> "FubolixConfig":
        if cfg.get("architecture") != "Fubolix" and "Fubolix" not in (cfg.get("architectures") or []):
            raise ConfigError(f"not a Fubolix config: architecture={cfg.get('architecture')!r}")
        layers = []
        for i, entry in enumerate(_need(cfg, "layers", "config.json")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"Fubolix config: {where} has the unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = dict(_need(entry, "mixer", where))
            if m.get("heads") is not None and m.get("kv_heads") is None:
                m["kv_heads"] = m["heads"]      # a file that leaves it out means one key head per head
            if m.get("dim") is not None and m.get("vdim") is None:
                m["vdim"] = m["dim"]            # ... and values as wide as keys
            for key in _REQUIRED[kind]:
                _need(m, key, where + ".mixer")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                m[key] = int(m[key])
                if m[key] < 1:
                    raise ConfigError(f"Fubolix config: {where}.mixer.{key} = {m[key]}")
            m["scale"] = float(m["scale"])
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"Fubolix config: {where}: {m['heads']} heads over {m['kv_heads']} key heads")
            if kind == "attention":
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"Fubolix config: {where}: the keys are the values, so dim ({m['dim']}) and vdim ({m['vdim']}) are one size")
                size = int(_need(m["mask"], "size", where + ".mixer.mask"))
                if size < 1:
                    raise ConfigError(f"Fubolix config: {where}.mixer.mask.size = {size}")
                m["mask"] = {"size": size, "keep_first": int(m["mask"].get("keep_first") or 0)}
            if kind in ("attention", "attention_3"):
                m["rot"] = _rot(m, where + ".mixer")
            if kind == "attention_2":
                qt = m.get("q_temp")
                if qt:
                    m["q_temp"] = {"coef": float(_need(qt, "coef", where + ".mixer.q_temp")),
                                   "every": float(_need(qt, "every", where + ".mixer.q_temp"))}
                    if m["q_temp"]["every"] <= 0:
                        raise ConfigError(f"Fubolix config: {where}.mixer.q_temp.every = {qt['every']}")
                else:
                    m["q_temp"] = None
            if kind == "attention_3":
                m["conv"] = int(m["conv"])
                if m["conv"] < 1:
                    raise ConfigError(f"Fubolix config: {where}.mixer.conv = {m['conv']} taps")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"Fubolix config: {where} has the unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(FubolixLayer(kind, m, None if mlp is None else int(_need(mlp, "ff", where + ".mlp"))))
        if not layers:
            raise ConfigError("Fubolix config: no layers")
        eos = (generation or {}).get("eos_token_id", cfg.get("eos_token_id"))
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=int(_need(cfg, "vocab", "config.json")), width=int(_need(cfg, "width", "config.json")),
                   eps=float(_need(_need(cfg, "norm", "config.json"), "eps", "norm")), layers=tuple(layers),
                   embedding_scale=float((cfg.get("embedding") or {}).get("scale") or 1.0), eos_token_ids=eos_ids)

    def to_hf(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
            "embedding": {"scale": self.embedding_scale}, "layers": [layer.to_hf() for layer in self.layers],
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
