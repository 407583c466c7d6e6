"""The Debuvik parts on the GPU against the plain statement in plain_debuvik.py: each mechanism alone, whole prompts against
token-by-token decoding, portions down to two tokens, unequal batches, pages that are used again, keys just inside and just
outside a chunk (in prompts and in decoding), a key far back, the first tokens, long decoding, sizes that differ everywhere
(also those that the tensor-core kernels take), and greedy generation through the engine.  Each test makes its own small
configuration and weights."""

from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import plain_debuvik as plain

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16

# ---- configurations ---------------------------------------------------------------------------------------------------

BANDS = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}  # with base 10000 and 8 pairs: kept, blended and slowed pairs


def latent(mlp=None, heads=3, dim=8, vdim=6, rank=16, scale=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale if scale is not None else dim ** -0.5}}


def attention(mlp=None, heads=4, kv_heads=2, dim=8, vdim=6, size=7, dims=4, base=10000.0, scaling=BANDS, softcap=5.0, scale=None,
              kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if size:
        m["mask"] = {"size": size}
    if dims is not None:
        m["rot"] = {"dims": dims, "base": base}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    if softcap:
        m["softcap"] = softcap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers, width=40, vocab=89, side=3, eps=1e-5):
    cfg = {"architecture": "Debuvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def full_config(**kw):
    """Both mixers, a layer on another's keys and values, layers with and without a feed-forward; sizes differ from layer to layer."""
    layers = [latent(dense(56), heads=2, dim=12, vdim=10, rank=24),
              attention(dense(24), heads=6, kv_heads=2, dim=16, vdim=4, size=9, dims=16),
              attention(None, heads=2, kv_heads=2, dim=16, vdim=4, size=5, dims=16, kv_from=1, softcap=2.0),
              latent(None, heads=5, dim=4, vdim=8, rank=12),
              attention(dense(16), heads=3, kv_heads=1, dim=6, vdim=10, size=11, dims=2, scaling=None)]
    return config(layers, **kw)


def random_weights(cfg: dict, seed: int, q_gain: float = 1.0) -> dict[str, torch.Tensor]:
    """Names and shapes from the framework's own list, values from here, bfloat16-representable."""
    from nanospec_b200.weights import build_model

    model, _ = build_model(cfg, None, F32, "cpu")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in sorted(model.weight_specs().items()):
        t = torch.randn(spec.shape, generator=g)
        leaf = name.split(".")[-1]
        if name == "side.embed":
            t = 0.8 * t
        elif len(spec.shape) == 2:
            t = t * (1.5 / math.sqrt(spec.shape[1]))
            if leaf in ("q", "uk"):
                t = t * q_gain
        elif leaf.startswith("norm"):
            t = 1.0 + 0.2 * t
            if name.endswith("mix.q.norm"):
                t = t * q_gain
        else:
            t = 0.5 * t  # biases
        out[name] = t.to(BF16).float()
    return out


def write_folder(folder, cfg, weights):
    from nanospec_b200.weights import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {k: v.to(BF16) for k, v in weights.items()})
    return folder


def make(tmp_path, cfg, seed=0, dtype=F32, blocks=64, page=4, slots=4, q_gain=1.0, weights=None):
    from nanospec_b200 import load_model
    from nanospec_b200.engine.step import ModelRunner

    w = weights if weights is not None else random_weights(cfg, seed, q_gain)
    model = load_model(write_folder(tmp_path / f"m{seed}{'f' if dtype == F32 else 'b'}", cfg, w), device="cuda", dtype=dtype)
    return ModelRunner(model, num_blocks=blocks, block_size=page, max_requests=slots), w


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def run_cut(runner, req_id, ids, cuts):
    """One request alone, its tokens in portions of the given sizes (the rest one by one); logits of every position."""
    from nanospec_b200.engine.step import StepEntry

    runner.begin(req_id)
    rows, at, sizes = [], 0, list(cuts)
    while at < len(ids):
        n = min(sizes.pop(0) if sizes else 1, len(ids) - at)
        rows.append(runner.step([StepEntry(req_id, ids[at: at + n], list(range(n)))]).float().cpu())
        at += n
    runner.end(req_id)
    runner.manager.check()
    return torch.cat(rows)


def distance(got, want):
    """Per position: root mean square over the vocabulary of the difference, the mean taken off, over the logits' spread."""
    d = got.double() - want.double()
    return (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.double().std()


def rounding(cfg, w, ids, want, samples=6):
    """Per position: how far bfloat16 storage of the activations alone moves the plain logits: the largest of the rounding
    itself and of `samples` draws of a relative error of that size on every stored activation.  (With norms on the sublayers'
    outputs a position can hang on a branch that nearly cancels; one draw alone misses such positions as often as not.)"""
    worst = distance(plain.forward(cfg, w, ids, rounded=BF16), want)
    for seed in range(samples):
        g = torch.Generator().manual_seed(seed)
        draw = lambda t: t * (1.0 + (torch.rand(t.shape, generator=g, dtype=t.dtype) - 0.5) * 2.0 ** -7)
        worst = torch.maximum(worst, distance(plain.forward(cfg, w, ids, rounded=draw), want))
    return worst


def close(got, want, dtype, what="", noise=None):
    """float32: a few roundings against the logits' spread at every position.  bfloat16: small at the median position, and at
    every position within a few times of what rounding alone does there (`noise`, from `rounding`; positions whose softmax
    hangs on one score amplify it), never of the size that a wrong mask, a lost bias or a wrong page gives elsewhere."""
    r = distance(got, want)
    if dtype == F32:
        assert float(r.max()) <= 2e-4, f"{what}: {float(r.max())} at position {int(r.argmax())} (limit 2e-4)"
        return
    noise = torch.zeros_like(r) if noise is None else noise[: len(r)]
    median, typical = float(r.median()), float(noise.median())
    assert median <= max(0.06, 3 * typical) or len(r) < 8, f"{what}: {median:.3f} at the median position (rounding alone: {typical:.3f})"
    over = r - torch.maximum(torch.full_like(r, 0.25), 4 * noise)
    assert float(over.max()) <= 0, f"{what}: {float(r[over.argmax()]):.3f} at position {int(over.argmax())} (rounding alone: {float(noise[over.argmax()]):.3f})"


# ---- the kernels alone ----------------------------------------------------------------------------------------------------

def test_norm_add_kernel_alone():
    """resid += rmsnorm(branch + bias) * gain and the stream's copy, at widths that take each of the kernel's forms."""
    from nanospec_b200 import ops

    g = torch.Generator().manual_seed(1)
    for H, with_bias in ((24, False), (33, True), (192, True), (1024, False), (2048, True), (4104, True), (5000, False)):
        N = 5
        resid, gain = torch.randn(N, H, generator=g), 1.0 + 0.3 * torch.randn(H, generator=g)
        bias = torch.randn(H, generator=g) if with_bias else None
        for dtype in (F32, BF16):
            y = torch.randn(N, H, generator=g).to(dtype)
            yb = y.double() + (bias.double() if with_bias else 0.0)
            want = resid.double() + plain.rms_norm(yb, gain.double(), 1e-5)
            r = resid.cuda().contiguous()
            cast = torch.empty(N, H, dtype=dtype, device="cuda")
            ops.norm_add(r, y.cuda(), gain.cuda(), 1e-5, cast=cast, bias=bias.cuda() if with_bias else None)
            assert (r.cpu() - want).abs().max() <= 1e-5 * float(want.abs().max()), (H, dtype)
            assert torch.equal(cast.cpu(), r.cpu().to(dtype)), (H, dtype)
            # without a branch: only the copy
            r2 = resid.cuda().contiguous()
            ops.norm_add(r2, None, None, 0.0, cast=cast)
            assert torch.equal(r2.cpu(), resid) and torch.equal(cast.cpu(), resid.to(dtype))


def test_small_kernels_alone():
    """The token's gated slice, the gate on rows, the bias on rows."""
    from nanospec_b200 import ops

    g = torch.Generator().manual_seed(2)
    N, dim, V = 9, 5, 17
    for dtype in (F32, BF16):
        tol = 1e-6 if dtype == F32 else 1e-2
        a = torch.randn(N, dim + 3, generator=g).to(dtype)
        table = torch.randn(V, 4 * dim, generator=g).to(dtype)
        ids = torch.randint(0, V, (N,), generator=g).int()
        out = ops.token_gate(a.cuda()[:, 2: 2 + dim], table.cuda(), ids.cuda(), 2 * dim, torch.empty(N, dim, dtype=dtype, device="cuda"))
        want = plain.gelu_tanh(a[:, 2: 2 + dim].double()) * table[ids.long()][:, 2 * dim: 3 * dim].double()
        assert (out.float().cpu() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
        x, z = torch.randn(N, 12, generator=g).to(dtype), torch.randn(N, 30, generator=g).to(dtype)
        got = ops.sigmoid_mul(x.cuda().clone(), z.cuda()[:, 7:19])
        assert (got.float().cpu() - x.double() * torch.sigmoid(z[:, 7:19].double())).abs().max() <= tol * 4
        b = torch.randn(12, generator=g)
        got = ops.add_bias(x.cuda().clone(), b.cuda())
        assert (got.float().cpu() - (x.double() + b.double())).abs().max() <= tol * 4


def test_banded_frequencies():
    """Every band of the frequency scaling is met, and the framework's frequencies are the plain ones."""
    from nanospec_b200.parts.position import rotary_frequencies

    rot = {"dims": 16, "base": 10000.0, "scaling": BANDS}
    f = plain.banded_frequencies(rot)
    raw = plain.banded_frequencies({"dims": 16, "base": 10000.0})
    ratio = (raw / f).tolist()
    assert any(abs(r - 1.0) < 1e-12 for r in ratio) and any(abs(r - 4.0) < 1e-9 for r in ratio) and any(1.01 < r < 3.99 for r in ratio)
    got, mag = rotary_frequencies(16, 10000.0, BANDS)
    assert mag == 1.0 and (got.double() - f).abs().max() <= 1e-7 * float(f.max())


def _paged(k, page, pages, generator):
    """[T, G, d] rows scattered over pages in a shuffled order: ([pages, G, page, d], table [1, blocks])."""
    T, G, d = k.shape
    blocks = -(-T // page)
    order = torch.randperm(pages, generator=generator)[:blocks]
    store = torch.zeros(pages, G, page, d, dtype=k.dtype)
    for t in range(T):
        store[order[t // page], :, t % page] = k[t]
    return store, order.int().view(1, -1)


@pytest.mark.parametrize("d,dv,H,G,chunk,cap", [(64, 32, 8, 2, 80, 25.0), (128, 128, 4, 4, 50, 0.0), (32, 80, 6, 1, 0, 4.0), (16, 16, 2, 2, 33, 1.5),
                                                 (64, 64, 3, 3, 200, 0.0), (24, 72, 4, 2, 40, 3.0), (120, 8, 2, 1, 65, 0.0)])
def test_attention_kernels_with_chunks_and_capped_scores(d, dv, H, G, chunk, cap):
    """The exact kernel (both precisions) and the two tensor-core kernels (a prompt's portion on top of cached keys, single
    tokens) against a plain softmax with the chunk mask and the cap, with one key made to dominate just inside the chunk
    of some queries, which a mask one position off or scores without the cap would show.  Values as wide as the keys, narrower
    and wider, in multiples of 16 and of 8."""
    from types import SimpleNamespace

    from nanospec_b200 import ops
    from nanospec_b200.parts.context import Workspace

    g = torch.Generator().manual_seed(d + H)
    T, page, pages = 333, 16, 40
    scale = d ** -0.5
    q = torch.randn(T, H, d, generator=g)
    k = torch.randn(T, G, d, generator=g)
    v = torch.randn(T, G, dv, generator=g)
    if chunk:
        # the first key of the chunks is what the queries that end them look for: inside for them, outside for the chunk before
        for c0 in range(0, T - 1, chunk):
            last = min(c0 + chunk, T) - 1
            k[c0] = 4.0 * q[last, 0] / q[last, 0].norm() * math.sqrt(d)
            if c0:
                q[c0 - 1, 0] = q[last, 0]  # the query just before the chunk would love that key and must not see it
    q, k, v = q.to(BF16).float(), k.to(BF16).float(), v.to(BF16).float()
    s = torch.einsum("ihd,jhd->hij", q.double(), k.double().repeat_interleave(H // G, 1)) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    p = plain.softmax_rows(s, plain.chunk_mask(T, chunk or None))
    want = torch.einsum("hij,jhe->ihe", p, v.double().repeat_interleave(H // G, 1)).reshape(T, H * dv)
    if chunk:  # the test tells a mask one key off apart
        p2 = plain.softmax_rows(s, plain.chunk_mask(T, chunk + 1))
        other = torch.einsum("hij,jhe->ihe", p2, v.double().repeat_interleave(H // G, 1)).reshape(T, H * dv)
        assert (other - want).abs().max() > 0.5
    for dtype in (F32, BF16):
        g2 = torch.Generator().manual_seed(d + H + 1)
        ks, table = _paged(k.to(dtype), page, pages, g2)
        g2 = torch.Generator().manual_seed(d + H + 1)
        vs, _ = _paged(v.to(dtype), page, pages, g2)
        ks, vs, table = ks.cuda(), vs.cuda(), table.cuda()
        qd = q.reshape(T, H * d).to(dtype).cuda()
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        req = torch.zeros(T, dtype=torch.int32, device="cuda")
        out = torch.zeros(T, H * dv, dtype=dtype, device="cuda")
        ops.attention_generic(qd, ks, vs, table, req, pos, out, H, G, d, page, scale, v_dim=dv, chunk=chunk, softcap=cap)
        tol = 2e-5 if dtype == F32 else 0.03
        assert (out.float().cpu() - want).abs().max() <= tol * float(want.abs().max()), ("exact", dtype)
    # the tensor-core kernels: positions 0 .. start-1 are cached, a portion of the rest, and single tokens at every edge
    lane = SimpleNamespace(k=ks, v=vs, block_table=table, page_size=page)
    for start, n in ((0, T), (100, 200), (chunk - 1 if chunk else 5, 130)):
        tiles = torch.tensor([[0, off] for off in range(0, n, ops.TILE_Q)], dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(positions=pos[start: start + n].contiguous(), qo_indptr=torch.tensor([0, n], dtype=torch.int32, device="cuda"))
        out = torch.zeros(n, H * dv, dtype=BF16, device="cuda")
        ops.attention_prefill(qd[start: start + n].contiguous(), lane, ctx, out, H, G, d, scale, 0, tiles, None, chunk=chunk, softcap=cap, v_dim=dv)
        torch.cuda.synchronize()
        assert (out.float().cpu() - want[start: start + n]).abs().max() <= 0.03 * float(want.abs().max()), ("prefill", start, n)
    rows = [0, 1, T - 1] + ([c for c in (chunk - 1, chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 3 * chunk) if 0 < c < T] if chunk else [77, 200])
    for n_splits_hint in (None, 64):
        B = len(rows)
        ctx = SimpleNamespace(positions=torch.tensor(rows, dtype=torch.int32, device="cuda"), token_req=torch.arange(B, dtype=torch.int32, device="cuda"),
                              qo_indptr=torch.arange(B + 1, dtype=torch.int32, device="cuda"), workspace=Workspace(torch.device("cuda")))
        lane_b = SimpleNamespace(k=ks, v=vs, block_table=table.repeat(B, 1).contiguous(), page_size=page)
        out = torch.zeros(B, H * dv, dtype=BF16, device="cuda")
        ops.attention_decode(qd[rows].contiguous(), lane_b, ctx, out, H, G, d, scale, 0, None, B, n_splits_hint, chunk=chunk, softcap=cap, v_dim=dv)
        torch.cuda.synchronize()
        assert (out.float().cpu() - want[rows]).abs().max() <= 0.03 * float(want.abs().max()), ("decode", n_splits_hint)


# ---- each mechanism alone -----------------------------------------------------------------------------------------------

SINGLE = {
    "latent attention alone": lambda: config([latent()], side=0),
    "one latent head, values wider than the latent": lambda: config([latent(heads=1, dim=6, vdim=20, rank=5)], side=0),
    "nine latent heads, a latent of 70": lambda: config([latent(heads=9, dim=4, vdim=12, rank=70)], side=0),
    "attention alone": lambda: config([attention()], side=0),
    "attention without a mask, a cap or a rotation": lambda: config([attention(size=0, softcap=0, dims=None)], side=0),
    "chunks of one": lambda: config([attention(size=1, heads=2, kv_heads=1)], side=0),
    "every query head with keys of its own, whole heads turn": lambda: config([attention(heads=3, kv_heads=3, dim=8, dims=8)], side=0),
    "three query heads to a key head, plain frequencies": lambda: config([attention(heads=6, kv_heads=2, dims=6, scaling=None, base=300.0)], side=0),
    "one head, values wider than keys": lambda: config([attention(heads=1, kv_heads=1, dim=4, vdim=18, dims=2, size=13)], side=0),
    "borrowed keys and values": lambda: config([attention(dense(16), size=6), latent(), attention(None, heads=2, size=4, softcap=0, kv_from=0)], side=0),
    "borrowed by two layers, one without a mask": lambda: config([attention(size=6), attention(size=0, kv_from=0), attention(heads=6, size=9, kv_from=0)], side=0),
    "feed-forward": lambda: config([latent(dense(24))], side=0),
    "side input": lambda: config([latent(), attention(dense(16))], side=5),
    "side input of one column": lambda: config([attention(None)], side=1),
    "everything": full_config,
}


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mechanism(name, dtype, tmp_path):
    """Whole, token by token and in portions (down to two tokens), against the plain statement."""
    cfg = SINGLE[name]()
    runner, w = make(tmp_path, cfg, seed=len(name), dtype=dtype)
    ids = tokens(37, cfg["vocab"], 5)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want)
    for cuts in ([37], [], [2, 3, 2, 11, 5, 2], [20, 1, 1, 15]):
        close(run_cut(runner, 0, ids, cuts), want, dtype, f"{name}, portions {cuts or 'of one'}", noise)


def test_layers_one_by_one(tmp_path):
    """The stream after every layer, in float32, against the plain statement's."""
    from nanospec_b200.engine.step import StepEntry

    cfg = full_config()
    runner, w = make(tmp_path, cfg, seed=3)
    ids = tokens(29, cfg["vocab"], 8)
    want, single = [], []
    plain.forward(cfg, w, ids, want)
    plain.F = F32  # the same statement in float32: what 32-bit rounding alone does to each layer's stream
    try:
        plain.forward(cfg, w, ids, single)
    finally:
        plain.F = torch.float64
    got = []
    runner.begin(0)
    ctx, rows, _ = runner.build_context([StepEntry(0, ids, [])])
    ctx.extras["probe"] = lambda i, resid, pending: got.append(resid.detach().cpu().double().clone())
    runner.forward(ctx, rows)
    runner.end(0)
    assert len(got) == len(want)
    for i, (a, b, c) in enumerate(zip(got, want, single)):
        limit = max(1e-5 * float(b.abs().max()), 3 * float((c.double() - b).abs().max()))
        assert (a - b).abs().max() <= limit, f"layer {i}: {float((a - b).abs().max())} (limit {limit})"


# ---- chunk edges, the cap, the biases, a key far back ---------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("dim,q_gain", [(8, 6.0), (16, 14.0)], ids=["exact", "tensor-core"])
def test_chunk_edges_the_cap_and_the_biases(dim, q_gain, dtype, tmp_path):
    """Queries are made large so that single scores decide the output: a chunk one key longer or shorter, scores without
    their cap, a lost bias or the lender's mask on the borrowing layer move the plain logits by far more than the engine
    differs from the right ones - in a prompt, in portions that cut through chunks and pages, and token by token.  Heads of
    8 run in the exact kernel in both types, heads of 16 in the tensor-core kernels in bfloat16."""
    size = 9
    cfg = config([attention(dense(16), heads=4, kv_heads=2, dim=dim, vdim=dim, size=size, dims=4, softcap=3.0),
                  attention(None, heads=4, kv_heads=2, dim=dim, vdim=dim, size=size - 4, dims=4, softcap=6.0, kv_from=0)], side=2)
    w = random_weights(cfg, 13, q_gain=q_gain)
    w["l1.mix.q.b"] = (32.0 * w["l1.mix.q.b"]).to(BF16).float()  # (the whole-projection norm shrinks what a bias of usual size does)
    runner, w = make(tmp_path, cfg, seed=14, dtype=dtype, page=4, weights=w)
    ids = tokens(45, cfg["vocab"], 17)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want)
    calm = noise <= 0.05  # bfloat16: the variants are told apart at the positions that rounding leaves alone
    wrong = []
    for li, base in ((0, size), (1, size - 4)):
        for delta in (-1, 1):
            other = copy.deepcopy(cfg)
            other["layers"][li]["mixer"]["mask"]["size"] = base + delta
            wrong.append(plain.forward(other, w, ids))
        other = copy.deepcopy(cfg)
        del other["layers"][li]["mixer"]["softcap"]
        wrong.append(plain.forward(other, w, ids))
    for name in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l0.mix.o.b", "l1.mix.q.b"):
        lost = dict(w)
        lost[name] = torch.zeros_like(w[name])
        wrong.append(plain.forward(cfg, lost, ids))
    for cuts in ([45], [], [size - 1, 2, size, 3, 2, 2, size + 1], [4, 4, 4, 4, 4], [size, size, size]):
        got = run_cut(runner, 0, ids, cuts)
        close(got, want, dtype, f"chunk edges, portions {cuts or 'of one'}", noise)
        keep = torch.ones_like(calm) if dtype == F32 else calm
        right = float(distance(got, want)[keep].max())
        for i, z in enumerate(wrong):
            off = float(distance(got, z)[keep].max())
            assert off > (10 if dtype == F32 else 3) * right and off > 0.03, f"variant {i} is not told apart: {off} against {right}"


def far_key_case():
    """One layer of latent attention whose last token looks for one token far back.  The queries are the keys' own map of
    the stream with its halves swapped (W_q = gain * W_uk W_dkv S, S the swap), and token 49's embedding is token 48's with
    the halves swapped: 49's query is 48's key direction, so the last position (a 49) puts its weight on the only 48."""
    width = 80  # (a latent of 64: among 450 random keys none comes near the one that is looked for)
    cfg = config([latent(heads=2, dim=32, vdim=8, rank=64)], width=width, side=0, vocab=50)
    w = random_weights(cfg, 41)
    uk, dkv = w["l0.mix.uk"].double(), w["l0.mix.dkv"].double()
    w["l0.mix.q"] = (4.0 * torch.roll(uk @ dkv, width // 2, dims=1)).to(BF16).float()
    w["embed"][49] = torch.roll(w["embed"][48], width // 2)
    ids = tokens(450, 48, 42)
    ids[31], ids[-1] = 48, 49          # 48 occurs nowhere else; position 31 is the last of the second page of 16
    lost = list(ids)
    lost[31] = 47
    return cfg, w, ids, lost


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
def test_a_key_far_back(dtype, tmp_path):
    """Latent attention sees every earlier key: the last token's query looks for one token 418 positions back, and a model
    that had lost that key would answer otherwise - in a whole prompt, as a decoded token and in portions."""
    cfg, w, ids, lost = far_key_case()
    runner, w = make(tmp_path, cfg, seed=41, dtype=dtype, page=16, blocks=40, weights=w)
    want = plain.forward(cfg, w, ids)
    assert float(distance(plain.forward(cfg, w, lost)[-1:], want[-1:]).max()) > 0.5
    for cuts in ([450], [449], [200, 100, 2, 140]):
        got = run_cut(runner, 0, ids, cuts)
        assert float(distance(got[-1:], want[-1:]).max()) <= (2e-4 if dtype == F32 else 0.1), cuts


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
def test_the_first_tokens_and_one_token_requests(dtype, tmp_path):
    cfg = full_config()
    runner, w = make(tmp_path, cfg, seed=21, dtype=dtype)
    for n in (1, 2, 3):
        ids = tokens(n, cfg["vocab"], 30 + n)
        want = plain.forward(cfg, w, ids)
        noise = rounding(cfg, w, ids, want)
        close(run_cut(runner, n, ids, [n]), want, dtype, f"a prompt of {n}", noise)
        close(run_cut(runner, n, ids, []), want, dtype, f"a prompt of {n}, token by token", noise)


def test_long_decoding(tmp_path):
    cfg = full_config()
    runner, w = make(tmp_path, cfg, seed=23, blocks=40, page=4)
    ids = tokens(150, cfg["vocab"], 24)
    close(run_cut(runner, 0, ids, [5]), plain.forward(cfg, w, ids), F32, "long decoding")


# ---- batches, pages that are used again -------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [31, 32])
def test_unequal_batches_and_reuse(seed, dtype, tmp_path):
    """Up to four requests of unequal lengths side by side, portions of some beside single tokens of others, on a pool
    that only their peak fits, requests ending and new ones taking their pages: every position as alone."""
    from nanospec_b200.engine.step import StepEntry

    cfg = full_config(side=3 if seed == 31 else 0)
    runner, w = make(tmp_path, cfg, seed=seed, dtype=dtype, blocks=30, page=4, slots=4)
    g = torch.Generator().manual_seed(seed)
    lengths = [23, 5, 41, 2, 17, 30, 9]
    prompts = [tokens(n, cfg["vocab"], seed * 100 + i) for i, n in enumerate(lengths)]
    want = [plain.forward(cfg, w, p) for p in prompts]
    got = [[] for _ in prompts]
    at = [0] * len(prompts)
    waiting, live = list(range(len(prompts))), []
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            runner.begin(live[-1])
        entries = []
        for i in live:
            left = len(prompts[i]) - at[i]
            n = min(left, int(torch.randint(1, 9, (1,), generator=g)))
            if left > 6 and torch.rand(1, generator=g) < 0.2:
                continue  # left out of this step, goes on later
            entries.append((i, n))
        if not entries:
            continue
        logits = runner.step([StepEntry(i, prompts[i][at[i]: at[i] + n], list(range(n))) for i, n in entries]).float().cpu()
        row = 0
        for i, n in entries:
            got[i].append(logits[row: row + n])
            row += n
            at[i] += n
            if at[i] == len(prompts[i]):
                runner.end(i)
                live.remove(i)
        runner.manager.check()
    for i in range(len(prompts)):
        close(torch.cat(got[i]), want[i], dtype, f"request {i} in a batch", rounding(cfg, w, prompts[i], want[i]) if dtype == BF16 else None)


# ---- other sizes, drawn from seeds ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_from_seeds(seed, tmp_path):
    g = torch.Generator().manual_seed(2000 + seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    layers, lenders = [], []
    for i in range(pick([2, 3, 5])):
        mlp = pick([None, dense(pick([8, 20, 64]))])
        kind = pick(["latent", "attention", "attention"])
        if kind == "latent":
            layers.append(latent(mlp, heads=pick([1, 2, 3, 7]), dim=pick([2, 8, 12, 32]), vdim=pick([2, 8, 20]), rank=pick([4, 16, 36, 64]),
                                 scale=pick([None, 0.3, 0.05])))
            continue
        dim = pick([2, 8, 12, 32])
        kw = dict(size=pick([0, 1, 3, 8, 33]), dims=pick([None, 0, 2, dim]), base=pick([100.0, 50000.0]), scaling=pick([None, BANDS]),
                  softcap=pick([0, 1.0, 20.0]), scale=pick([None, 0.6, 0.11]))
        if lenders and pick([True, False]):
            src = pick(lenders)
            sm = layers[src]["mixer"]
            layers.append(attention(mlp, heads=sm["kv_heads"] * pick([1, 2]), kv_heads=sm["kv_heads"], dim=sm["dim"], vdim=sm["vdim"],
                                    kv_from=src, **{**kw, "dims": (sm.get("rot") or {}).get("dims"), "base": (sm.get("rot") or {"base": 1.0})["base"],
                                                    "scaling": (sm.get("rot") or {}).get("scaling")}))
        else:
            kv = pick([1, 2, 3])
            layers.append(attention(mlp, heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=dim, vdim=pick([2, 8, 20, dim]), **kw))
            lenders.append(i)
    cfg = config(layers, width=pick([16, 24, 72]), vocab=pick([50, 131]), side=pick([0, 1, 4]), eps=pick([1e-5, 1e-6, 1e-3]))
    for dtype in (F32, BF16):
        runner, w = make(tmp_path, cfg, seed=seed, dtype=dtype, page=pick([2, 4, 16]))
        ids = tokens(48, cfg["vocab"], seed)
        want = plain.forward(cfg, w, ids)
        noise = rounding(cfg, w, ids, want)
        for cuts in ([48], [7, 2, 2, 19, 3], []):
            close(run_cut(runner, 0, ids, cuts), want, dtype, f"seed {seed}, portions {cuts or 'of one'}: {json.dumps(cfg)[:300]}", noise)


@pytest.mark.parametrize("dim,vdim,heads,kv_heads,size,rank", [(64, 32, 8, 2, 88, 48), (128, 128, 4, 4, 70, 128), (32, 64, 6, 1, 130, 96),
                                                                (16, 16, 4, 2, 40, 256), (40, 24, 2, 1, 75, 32)])
def test_tensor_core_sizes(dim, vdim, heads, kv_heads, size, rank, tmp_path):
    """Head sizes and latents that the tensor-core attention kernels take (values as wide as keys, narrower, wider), in bfloat16, over prompts
    long enough for several key tiles and chunks, with portions and single tokens; float32 beside it."""
    cfg = config([attention(dense(64), heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, size=size, dims=dim // 2, softcap=8.0),
                  latent(None, heads=heads, dim=16, vdim=16, rank=rank),
                  attention(None, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, size=size + 5, dims=dim // 2, softcap=0, kv_from=0)],
                 width=64, side=4)
    ids = tokens(300, cfg["vocab"], rank)
    w = random_weights(cfg, rank)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want)
    for dtype in (BF16, F32):
        runner, _ = make(tmp_path, cfg, seed=rank, dtype=dtype, blocks=64, page=16, weights=w)
        for cuts in ([300], [130, 2, 67, 64] + [1] * 20 + [17]):
            close(run_cut(runner, 0, ids, cuts), want, dtype, f"head size {dim}, portions {cuts[:4]}", noise)


# ---- through the engine: scheduler, graphs, sampling, command line ------------------------------------------------------------

@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_greedy_generation_through_the_engine(dtype, graphs, tmp_path):
    from nanospec_b200 import Engine, EngineConfig, SamplingParams, load_model

    cfg = full_config()
    w = random_weights(cfg, 71)
    model = load_model(write_folder(tmp_path / "gen", cfg, w), device="cuda", dtype=dtype)
    eng = Engine(model, EngineConfig(num_blocks=64, block_size=4, max_running=3, prefill_chunk=11, cuda_graphs=graphs,
                                     graph_buckets=(1, 2, 4)))
    prompts = [tokens(n, cfg["vocab"], 80 + n) for n in (3, 30, 1, 17, 12)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    for p, out in zip(prompts, outs):
        assert len(out) == 12
        z = plain.forward(cfg, w, p + out)
        for j, tok in enumerate(out):
            row = z[len(p) + j - 1]
            gap = float(row.max() - row[tok]) / float(z.std())
            assert gap <= (1e-3 if dtype == F32 else 0.1), f"token {j}: another token is ahead by {gap} of the logits' spread"


def test_command_line(tmp_path):
    """Random weights from a config.json, seeded sampling twice the same, greedy generation in float32, a trace replayed."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(full_config()))
    run = lambda *a, **kw: subprocess.run([sys.executable, "-m", "nanospec_b200", *a], cwd=root, capture_output=True, text=True, timeout=600, **kw)
    r = run("random-weights", "--config", str(cfg_path), "--out", str(tmp_path / "model"), "--seed", "4")
    assert r.returncode == 0, r.stderr
    outs = []
    for _ in range(2):
        r = run("generate", "--model", str(tmp_path / "model"), "--prompt-lens", "5", "21", "--max-tokens", "9", "--temperature", "0.8",
                "--top-k", "20", "--top-p", "0.9", "--seed", "3", "--ignore-eos")
        assert r.returncode == 0, r.stderr
        outs.append([json.loads(line)["output_ids"] for line in r.stdout.splitlines() if '"output_ids"' in line])
    assert outs[0] == outs[1] and [len(o) for o in outs[0]] == [9, 9]
    r = run("generate", "--model", str(tmp_path / "model"), "--dtype", "float32", "--prompt-ids", "1 2 3 4", "--max-tokens", "6", "--ignore-eos")
    assert r.returncode == 0, r.stderr
    assert len(json.loads(r.stdout.splitlines()[0])["output_ids"]) == 6
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3, 4, 5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [6], "want": [0]}, {"id": "b", "tokens": [7, 8], "want": []}], "end": ["a"]}]
    r = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path / "model"), "--dtype", "float32", "--out", str(tmp_path / "o"),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "done 0" in r.stdout and "done 1" in r.stdout, r.stderr
    assert (tmp_path / "o" / "0.f32").stat().st_size == 4 * full_config()["vocab"]
