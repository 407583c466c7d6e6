"""The Debuvik configuration, its recipe, lanes and tensor names, and the plain statement against itself; no GPU."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_debuvik as plain
import nanospec_b200.architectures  # noqa: F401  (registers the architectures)
from nanospec_b200.config import ConfigError, resolve_architecture
from nanospec_b200.config.debuvik import DebuvikConfig
from nanospec_b200.weights import build_model


def _attention(**kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "softcap": 5.0, "mask": {"size": 7},
         "rot": {"dims": 4, "base": 1000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}
    m.update(kw)
    return m


def _cfg():
    latent = {"heads": 3, "dim": 8, "vdim": 10, "kv_rank": 12, "scale": 0.25}
    layers = [{"type": "latent_attention", "mixer": latent, "mlp": {"kind": "dense", "ff": 20}},
              {"type": "attention", "mixer": _attention(), "mlp": {"kind": "dense", "ff": 12}},
              {"type": "latent_attention", "mixer": dict(latent, heads=2), "mlp": None},
              {"type": "attention", "mixer": _attention(heads=2, kv_from=1, mask={"size": 3}), "mlp": None},
              {"type": "attention", "mixer": _attention(kv_heads=1, vdim=8), "mlp": {"kind": "dense", "ff": 8}}]
    return {"architecture": "Debuvik", "vocab": 53, "width": 24, "norm": {"eps": 1e-5}, "token_side": {"dim": 3}, "layers": layers}


def test_round_trip_and_registry():
    cfg = DebuvikConfig.from_hf(_cfg())
    assert DebuvikConfig.from_hf(cfg.to_hf()) == cfg
    assert resolve_architecture(_cfg()).name == "Debuvik"
    assert cfg.side_dim == 3 and cfg.layers[3].kv_from == 1 and cfg.layers[1].kv_from is None and cfg.layers[2].ff is None
    bare = _cfg()
    del bare["token_side"]
    assert DebuvikConfig.from_hf(bare).side_dim == 0


def test_recipe_order_lanes_and_names():
    model, _ = build_model(_cfg(), None, torch.float32, "cpu")
    order = model.recipe.order
    # the fourth layer reads the second layer's lane and writes nothing; every other layer has a lane of its own
    assert [(r.layer, r.lane, r.writes) for r in order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False), (4, 3, True)]
    names = set(model.weight_specs())
    assert {"embed", "side.embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk",
            "l0.mix.uv", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l0.side.gate", "l0.side.proj", "l0.side.norm",
            "l1.mix.q", "l1.mix.q.b", "l1.mix.k", "l1.mix.k.b", "l1.mix.v", "l1.mix.v.b", "l1.mix.q.norm", "l1.mix.k.norm", "l1.mix.o",
            "l1.mix.o.b", "l3.mix.q", "l3.mix.q.b", "l3.mix.q.norm", "l3.mix.o", "l3.mix.o.b", "l3.side.norm"} <= names
    assert not any(n.startswith(("l3.mix.k", "l3.mix.v")) for n in names)   # no keys and values of its own
    assert "l2.norm2" not in names and not any(n.startswith(("l2.mlp", "l3.mlp")) for n in names)
    specs = model.weight_specs()
    assert specs["side.embed"].shape == (53, 5 * 3) and specs["l0.mix.g"].shape == (3 * 10, 24) and specs["l1.mix.q.norm"].shape == (32,)
    assert specs["l1.mix.v"].shape == (2 * 6, 24) and specs["l3.mix.o"].shape == (24, 2 * 6)
    needs = model.lane_needs()
    assert len(needs) == 4
    assert needs[0][0].kv_heads == 1 and needs[0][0].head_dim == 12 and needs[0][0].v_dim == 0          # the latent alone
    assert needs[1][0].kv_heads == 2 and needs[1][0].head_dim == 8 and needs[1][0].v_dim == 6           # values narrower than keys
    assert needs[3][0].kv_heads == 1 and needs[3][0].head_dim == 8 and needs[3][0].v_dim in (None, 8)
    assert all(n[0].window == 0 for n in needs)  # chunks keep every page: a borrower may be masked otherwise
    bare = _cfg()
    del bare["token_side"]
    model, _ = build_model(bare, None, torch.float32, "cpu")
    assert not any("side" in n for n in model.weight_specs())


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0].update(type="retention"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].update(heads=3), "query heads"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "chunks"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=3), "pairs"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "pairs"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "keys and values"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "keys and values"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=3), "keys and values"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "differ in size"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "feed-forward kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(token_side={}), "dim"),
])
def test_refusals(edit, text):
    cfg = _cfg()
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        DebuvikConfig.from_hf(cfg)


def _weights(cfg, seed=0):
    model, _ = build_model(cfg, None, torch.float32, "cpu")
    g = torch.Generator().manual_seed(seed)
    return {n: torch.randn(s.shape, generator=g) * (0.3 if len(s.shape) == 2 else 0.2) + (1.0 if n.split(".")[-1].startswith("norm") else 0.0)
            for n, s in model.weight_specs().items()}


def test_plain_statement_against_itself():
    """A token's logits do not depend on what follows it; chunks longer than the sequence are no chunks; a cap far above the
    scores is no cap; the layer that borrows keys sees the lender's, so the lender's key bias moves it."""
    cfg = _cfg()
    w = _weights(cfg)
    ids = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:9]), whole[:9], atol=1e-9)
    wide, wider = copy.deepcopy(cfg), copy.deepcopy(cfg)
    for a, size in ((wide, 23), (wider, 500)):
        for layer in a["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["mask"]["size"] = size
    assert torch.allclose(plain.forward(wide, w, ids), plain.forward(wider, w, ids), atol=1e-9)
    assert not torch.allclose(plain.forward(wide, w, ids), whole, atol=1e-6)
    high, none = copy.deepcopy(cfg), copy.deepcopy(cfg)
    for layer in high["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["softcap"] = 1e6
    for layer in none["layers"]:
        layer["mixer"].pop("softcap", None)
    assert torch.allclose(plain.forward(high, w, ids), plain.forward(none, w, ids), atol=1e-6)
    assert not torch.allclose(plain.forward(none, w, ids), whole, atol=1e-6)
    only = copy.deepcopy(cfg)
    only["layers"] = only["layers"][:4]
    w4 = {k: v for k, v in w.items() if not k.startswith("l4.")}
    streams, moved = [], []
    plain.forward(only, w4, ids, streams)
    plain.forward(only, dict(w4, **{"l1.mix.k.b": w4["l1.mix.k.b"] + 1.0}), ids, moved)
    assert not torch.allclose(moved[3] - moved[2], streams[3] - streams[2], atol=1e-6)


def test_plain_mechanisms():
    """The chunk mask, the rotation's layout and the frequency bands of the plain statement, each against its definition."""
    mask = plain.chunk_mask(10, 4)
    for i in range(10):
        for j in range(10):
            assert bool(mask[i, j]) == (j <= i and i // 4 == j // 4)
    assert bool(plain.chunk_mask(6, None)[5, 0])
    rot = {"dims": 4, "base": 100.0}
    x = torch.arange(1.0, 7.0, dtype=torch.float64).view(1, 1, 6)
    y = plain.rotate_half(x, torch.tensor([3]), rot)
    for i in range(2):  # feature i turns with feature i + 2 by 3 * 100^(-2i/4); features 4 and 5 pass
        a = 3.0 * 100.0 ** (-2.0 * i / 4)
        u, v = float(x[0, 0, i]), float(x[0, 0, i + 2])
        assert abs(float(y[0, 0, i]) - (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(float(y[0, 0, i + 2]) - (v * math.cos(a) + u * math.sin(a))) < 1e-12
    assert torch.equal(y[..., 4:], x[..., 4:])
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    f = plain.banded_frequencies({"dims": 16, "base": 10000.0, "scaling": sc})
    raw = plain.banded_frequencies({"dims": 16, "base": 10000.0})
    for a, b in zip(f.tolist(), raw.tolist()):
        wave = 2 * math.pi / b
        if wave < 16:
            assert a == b
        elif wave > 64:
            assert abs(a - b / 4) < 1e-15
        else:
            s = (64 / wave - 1.0) / 3.0
            assert abs(a - ((1 - s) * b / 4 + s * b)) < 1e-15
    z = torch.tensor([-2.0, 0.0, 0.7], dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-12)
