"""The Debuvik decoder as a recipe: layers that norm each sublayer's output ("outnorm") around attention over a cached
latent with a gate on every output feature, or grouped-query attention with biases, whole-projection q/k norms, partly
rotated heads, capped scores and a mask of chunks (on its own keys and values or on an earlier layer's lane), a gated
feed-forward or none, and the token's own gated side input; a final RMS norm and a head.  Tensor names: `embed`,
`side.embed`, `l<i>.mix.<name>`, `l<i>.norm1`, `l<i>.mlp.<name>`, `l<i>.norm2`, `l<i>.side.<name>`, `final.norm`, `head`."""

from __future__ import annotations

from ..config.debuvik import DebuvikConfig, MAX_POSITIONS
from ..config.recipe import LayerSpec, ModelRecipe, PartSpec, Run
from ..config.registry import Architecture, register_architecture


def _mixer(kind: str, m: dict, width: int, eps: float) -> PartSpec:
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden": width, "heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": 0, "v_dim": int(m["vdim"]),
            "rank": int(m["kv_rank"]), "scale": float(m["scale"]), "window": 0, "eps": eps, "sink": False, "gate": "feature",
            "position": None})
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    position = PartSpec("rotary", {"head_dim": int(m["dim"]), "dims": int(rot["dims"]), "base": float(rot["base"]),
                                   "layout": "half", "scaling": rot.get("scaling") or None})
    return PartSpec("gqa_attention", {
        "hidden": width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
        "v_dim": int(m["vdim"]), "scale": float(m["scale"]), "qk_norm": {"eps": eps}, "position": position,
        "chunk": int((m.get("mask") or {}).get("size") or 0), "softcap": float(m.get("softcap") or 0.0), "bias": True,
        "own_kv": m.get("kv_from") is None, "wide_weights": True,
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})


def debuvik_recipe(cfg: DebuvikConfig) -> ModelRecipe:
    norm = PartSpec("rmsnorm", {"hidden": cfg.width, "eps": cfg.eps, "weight_name": ""})
    names = {"mixer": "mix.", "feed_forward": "mlp.", "norm_mixer": "norm1", "norm_feed_forward": "norm2", "side_input": "side."}
    layers, order, lane_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        ff = None if layer.ff is None else PartSpec("swiglu", {"hidden": cfg.width, "intermediate": layer.ff,
                                                                "names": {"gate": "gate", "up": "up", "down": "down"}})
        params = {}
        if cfg.side_dim:
            params["side_input"] = PartSpec("token_gate", {"hidden": cfg.width, "dim": cfg.side_dim, "index": i, "eps": cfg.eps})
        layers.append(LayerSpec(block="outnorm", prefix=f"l{i}.", mixer=_mixer(layer.type, layer.mixer, cfg.width, cfg.eps),
                                feed_forward=ff, norm=norm, names=names, params=params))
        if layer.kv_from is None:  # a lane of its own; a layer that borrows keys and values reads the lender's
            lane_of[i] = len(lane_of)
            order.append(Run(layer=i, lane=lane_of[i]))
        else:
            order.append(Run(layer=i, lane=lane_of[layer.kv_from], writes=False))
    embedding = {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "embed"}
    if cfg.side_dim:
        embedding.update(side_name="side.embed", side_columns=cfg.side_dim * len(cfg.layers))
    return ModelRecipe(
        architecture=cfg.architecture, embedding=PartSpec("table", embedding),
        layers=tuple(layers), order=tuple(order), final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "head", "tied_to": None}),
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS, eos_token_ids=cfg.eos_token_ids)


DEBUVIK = register_architecture(Architecture(
    name="Debuvik", model_type="debuvik", config_from_hf=DebuvikConfig.from_hf, recipe=debuvik_recipe))
