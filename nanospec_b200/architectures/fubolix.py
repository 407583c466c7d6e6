"""The Fubolix decoder as a recipe: layers in the "parallel" arrangement (one dynamic-tanh norm whose output the mixer and the
feed-forward both read), a mixer of one of three kinds of grouped-query attention with a sink in the softmax's denominator, a
dense feed-forward with a squared relu or none, a scaled embedding, a final dynamic-tanh norm and a head.

    attention     keys that double as values, rotation of interleaved pairs (YaRN frequencies), q and k divided by their root mean
                  square per head after the rotation, a sliding window that keeps a sequence's first keys, a sink of score 0,
                  one sigmoid gate per head on the heads' outputs
    attention_2   q and k normed per head with a gain shared by the heads, no rotation, queries scaled by a factor that grows with
                  the logarithm of the position, every earlier key, a sink of score 0
    attention_3   a short causal convolution over time on q, k and v, rotation in halves (YaRN frequencies), every earlier key, a
                  learned sink per head

Tensor names: `embed`, `l<i>.norm1` (+ `.b`, `.alpha`), `l<i>.mix.{q, k, v, g, o, sink, q.norm, k.norm, q.conv, k.conv, v.conv}`,
`l<i>.mlp.{up, down}`, `final.norm` (+ `.b`, `.alpha`), `head`."""

from __future__ import annotations

from ..config.fubolix import FubolixConfig, MAX_POSITIONS
from ..config.recipe import LayerSpec, ModelRecipe, PartSpec, Run
from ..config.registry import Architecture, register_architecture

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "sink": "sink", "q_norm": "q.norm", "k_norm": "k.norm",
          "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}


def _mixer(kind: str, m: dict, width: int, eps: float) -> PartSpec:
    params = {"hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
              "scale": m["scale"], "wide_weights": True, "names": _NAMES, "position": None}
    if kind in ("attention", "attention_3"):
        rot = m["rot"]
        params["position"] = PartSpec("rotary", {"head_dim": m["dim"], "dims": rot["dims"], "base": rot["base"],
                                                 "layout": "interleaved" if kind == "attention" else "half",
                                                 "scaling": rot.get("scaling") or None})
    if kind == "attention":
        params.update(window=m["mask"]["size"], keep_first=m["mask"]["keep_first"], v_from_k=True, head_gate=True, sink="zero",
                      head_norm={"eps": eps, "when": "after", "gain": False})
    elif kind == "attention_2":
        params.update(sink="zero", head_norm={"eps": eps, "when": "before", "gain": True}, q_temp=m.get("q_temp"))
    else:
        params.update(sink="learned", conv=m["conv"])
    return PartSpec("gqa_attention", params)


def fubolix_recipe(cfg: FubolixConfig) -> ModelRecipe:
    norm = PartSpec("dyt", {"hidden": cfg.width, "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        ff = None if layer.ff is None else PartSpec("dense_act", {"hidden": cfg.width, "intermediate": layer.ff, "activation": "relu2",
                                                                   "names": {"up": "up", "down": "down"}})
        layers.append(LayerSpec(block="parallel", prefix=f"l{i}.", mixer=_mixer(layer.type, layer.mixer, cfg.width, cfg.eps),
                                feed_forward=ff, norm=norm, names={"mixer": "mix.", "feed_forward": "mlp.", "norm_mixer": "norm1"}))
    order = tuple(Run(layer=i, lane=i) for i in range(len(layers)))
    return ModelRecipe(
        architecture=cfg.architecture,
        embedding=PartSpec("table", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "embed",
                                     "scale": cfg.embedding_scale}),
        layers=tuple(layers), order=order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "", "weight_name": "head", "tied_to": None}),
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS, eos_token_ids=cfg.eos_token_ids)


FUBOLIX = register_architecture(Architecture(
    name="Fubolix", model_type="fubolix", config_from_hf=FubolixConfig.from_hf, recipe=fubolix_recipe))
