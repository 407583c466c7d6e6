"""The Fubolix configuration, its recipe, its tensor names and the plain statement's own mechanisms, without a GPU."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_fubolix as plain
import nanospec_b200.architectures  # noqa: F401  (registers the architectures)


def yarn(factor=4.0, original=64, fast=8.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def small_config():
    return {
        "architecture": "Fubolix", "vocab": 61, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
        "layers": [
            {"type": "attention_3", "mlp": None,
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "conv": 3, "rot": {"dims": 4, "base": 100.0, "scaling": yarn()}}},
            {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
             "mixer": {"heads": 6, "kv_heads": 3, "dim": 10, "vdim": 10, "scale": 0.2, "mask": {"size": 5, "keep_first": 2},
                       "rot": {"dims": 6, "base": 1000.0}}},
            {"type": "attention_2", "mlp": {"kind": "dense", "ff": 16},
             "mixer": {"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 4, "scale": 0.25, "q_temp": {"coef": 0.4, "every": 3}}},
        ]}


def test_config_round_trip_and_recipe():
    from nanospec_b200.config import FubolixConfig, resolve_architecture

    cfg = small_config()
    arch = resolve_architecture(cfg)
    assert arch.name == "Fubolix"
    typed = arch.config_from_hf(cfg, None)
    assert isinstance(typed, FubolixConfig) and typed.embedding_scale == 2.0 and typed.width == 24
    again = FubolixConfig.from_hf(typed.to_hf())
    assert again == typed
    recipe = arch.recipe(typed)
    assert [layer.block for layer in recipe.layers] == ["parallel"] * 3
    assert [run.lane for run in recipe.order] == [0, 1, 2] and all(run.writes for run in recipe.order)
    a3, a1, a2 = (layer.mixer.params for layer in recipe.layers)
    assert a3["sink"] == "learned" and a3["conv"] == 3 and a3["position"]["layout"] == "half" and not a3.get("v_from_k")
    assert a1["sink"] == "zero" and a1["v_from_k"] and a1["head_gate"] and a1["window"] == 5 and a1["keep_first"] == 2
    assert a1["head_norm"] == {"eps": 1e-5, "when": "after", "gain": False} and a1["position"]["layout"] == "interleaved"
    assert a2["sink"] == "zero" and a2["position"] is None and a2["head_norm"]["when"] == "before" and a2["head_norm"]["gain"]
    assert a2["q_temp"] == {"coef": 0.4, "every": 3.0}
    assert recipe.layers[0].feed_forward is None and recipe.layers[1].feed_forward["activation"] == "relu2"
    assert recipe.embedding["scale"] == 2.0 and recipe.final_norm.kind == "dyt"


def test_defaults_and_refusals():
    from nanospec_b200.config import ConfigError, FubolixConfig

    cfg = small_config()
    del cfg["embedding"]
    del cfg["layers"][2]["mixer"]["q_temp"]
    del cfg["layers"][2]["mixer"]["kv_heads"]
    typed = FubolixConfig.from_hf(cfg)
    assert typed.embedding_scale == 1.0 and typed.layers[2].mixer["q_temp"] is None and typed.layers[2].mixer["kv_heads"] == 2

    def broken(change):
        c = small_config()
        change(c)
        with pytest.raises(ConfigError) as err:
            FubolixConfig.from_hf(c)
        return str(err.value)

    assert "layers[1]" in broken(lambda c: c["layers"][1]["mixer"].pop("mask"))
    assert "unknown mixer type" in broken(lambda c: c["layers"][0].update(type="attention_9"))
    assert "key heads" in broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=4))
    assert "one size" in broken(lambda c: c["layers"][1]["mixer"].update(vdim=8))
    assert "rot" in broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=9))
    assert "scaling" in broken(lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"))
    assert "feed-forward kind" in broken(lambda c: c["layers"][1]["mlp"].update(kind="routed"))
    assert "every" in broken(lambda c: c["layers"][2]["mixer"]["q_temp"].update(every=0))
    assert "not a Fubolix config" in broken(lambda c: c.update(architecture="Other"))
    assert "norm" in broken(lambda c: c.pop("norm"))


def test_tensor_names_and_loader_errors(tmp_path):
    from nanospec_b200.weights import WeightError, build_model, load_model, write_random_model, write_safetensors
    from nanospec_b200.weights.safetensors_io import SafetensorsFile

    cfg = small_config()
    model, _ = build_model(cfg, None, torch.float32, "cpu")
    specs = model.weight_specs()
    assert specs["l0.norm1.alpha"].shape == () and specs["l0.norm1.b"].shape == (24,) and specs["final.norm.alpha"].shape == ()
    assert specs["l0.mix.q.conv"].shape == (32, 3) and specs["l0.mix.v.conv"].shape == (12, 3) and specs["l0.mix.sink"].shape == (4,)
    assert specs["l1.mix.g"].shape == (6, 24) and "l1.mix.v" not in specs and specs["l1.mix.o"].shape == (24, 60)
    assert specs["l2.mix.q.norm"].shape == (12,) and specs["l2.mix.k.norm"].shape == (12,) and specs["l2.mix.v"].shape == (4, 24)
    assert "l0.mlp.up" not in specs and specs["l1.mlp.up"].shape == (40, 24) and specs["l2.mlp.down"].shape == (24, 16)
    assert not any(".norm2" in n for n in specs)
    needs = model.lane_needs()
    assert needs[0][1].shape == (2 * (32 + 16 + 12),) and needs[1][1] is None and needs[1][0].keep_first == 2 and needs[2][0].v_dim == 4
    folder = write_random_model(tmp_path / "m", cfg, seed=3)
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {k: f.tensor(k).clone() for k in f.keys()}
    assert set(tensors) == set(specs)
    del tensors["l1.mix.g"]
    tensors["l1.mix.v"] = torch.zeros(30, 24, dtype=torch.bfloat16)
    tensors["l0.mix.sink"] = torch.zeros(5, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError) as err:
        load_model(folder, device="cpu", dtype=torch.float32)
    text = str(err.value)
    assert "l1.mix.g" in text and "l1.mix.v" in text and "l0.mix.sink" in text


# ---- the plain statement's own mechanisms: a second, independent writing of each ----------------------------------------

def test_plain_yarn_frequencies_meet_every_band():
    rot = {"dims": 16, "base": 10000.0, "scaling": yarn(factor=4.0, original=64, fast=8.0, slow=1.0)}
    f, mag = plain.yarn_frequencies(rot)
    raw, one = plain.yarn_frequencies({"dims": 16, "base": 10000.0})
    ratio = (raw / f).tolist()
    assert one == 1.0 and abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert abs(ratio[0] - 1.0) < 1e-12 and abs(ratio[-1] - 4.0) < 1e-9 and any(1.01 < x < 3.99 for x in ratio)
    from nanospec_b200.parts.position import rotary_frequencies

    got, got_mag = rotary_frequencies(16, 10000.0, rot["scaling"])
    assert abs(got_mag - mag) < 1e-12 and (got.double() - f).abs().max() <= 1e-7 * float(f.max())


def test_plain_rotation_layouts_and_partial_heads():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.arange(5)
    rot = {"dims": 4, "base": 50.0}
    for layout, pairs in (("interleaved", [(0, 1), (2, 3)]), ("half", [(0, 2), (1, 3)])):
        y = plain.rotate(x, pos, rot, layout)
        assert torch.equal(y[..., 4:], x[..., 4:]) and torch.allclose(y[0], x[0])
        for i, (a, b) in enumerate(pairs):
            ang = 3.0 * 50.0 ** (-2.0 * i / 4)
            assert abs(float(y[3, 1, a]) - (float(x[3, 1, a]) * math.cos(ang) - float(x[3, 1, b]) * math.sin(ang))) < 1e-12
            assert abs(float(y[3, 1, b]) - (float(x[3, 1, b]) * math.cos(ang) + float(x[3, 1, a]) * math.sin(ang))) < 1e-12


def test_plain_masks_sink_and_convolution():
    m = plain.window_mask(9, 3, 2)
    assert m[8].tolist() == [True, True, False, False, False, False, True, True, True]
    assert m[2].tolist() == [True, True, True] + [False] * 6 and not m[0, 1]
    s = torch.zeros(1, 2, 2, dtype=torch.float64)
    p = plain.softmax_with_sink(s, plain.causal_mask(2), torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(p[0], torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]], dtype=torch.float64))
    p = plain.softmax_with_sink(s, plain.causal_mask(2), torch.tensor([math.log(2.0)], dtype=torch.float64))
    assert torch.allclose(p[0, 1], torch.tensor([0.25, 0.25], dtype=torch.float64))
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None].repeat(1, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = plain.causal_convolution(u, w)
    assert y[:, 0].tolist() == [100.0, 210.0, 321.0, 432.0, 543.0] and y[:, 1].tolist() == [1.0, 2.0, 3.0, 4.0, 5.0]


def test_plain_forward_is_causal_and_uses_every_mechanism():
    """A later token never moves an earlier position, and taking a mechanism away moves the logits."""
    cfg = small_config()
    from nanospec_b200.weights import build_model

    model, _ = build_model(cfg, None, torch.float32, "cpu")
    g = torch.Generator().manual_seed(4)
    w = {n: (torch.randn(s.shape, generator=g) * (0.4 if len(s.shape) == 2 else 1.0)).to(torch.bfloat16).float() for n, s in sorted(model.weight_specs().items())}
    ids = torch.randint(0, 61, (14,), generator=g).tolist()
    z = plain.forward(cfg, w, ids)
    assert z.shape == (14, 61) and torch.isfinite(z).all()
    other = list(ids)
    other[9] = (other[9] + 1) % 61
    z2 = plain.forward(cfg, w, other)
    assert torch.equal(z2[:9], z[:9]) and not torch.allclose(z2[9:], z[9:])

    def without(change):
        c = copy.deepcopy(cfg)
        change(c)
        return float((plain.forward(c, w, ids) - z).abs().max())

    assert without(lambda c: c["layers"][1]["mixer"]["mask"].update(size=6)) > 1e-6
    assert without(lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=1)) > 1e-6
    assert without(lambda c: c["layers"][2]["mixer"].update(q_temp=None)) > 1e-6
    assert without(lambda c: c["layers"][0]["mixer"]["rot"].update(scaling=None)) > 1e-6
    assert without(lambda c: c.update(embedding={"scale": 1.0})) > 1e-6
    for name in ("l0.mix.sink", "l1.mix.g", "l0.mix.k.conv", "l2.mix.k.norm", "l1.norm1.b", "final.norm.alpha"):
        lost = dict(w)
        lost[name] = torch.zeros_like(w[name]) if "alpha" not in name else w[name] * 0.5
        assert float((plain.forward(cfg, lost, ids) - z).abs().max()) > 1e-6, name
