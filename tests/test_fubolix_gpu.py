"""The Fubolix parts on the GPU against the plain statement in plain_fubolix.py: each kernel and each mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, unequal batches, pages and state slots that are used
again, keys just inside and just outside a window and among the kept first ones (in prompts and in decoding), a key far
back, the first tokens, long decoding, sizes that differ everywhere (also those that the tensor-core kernels take), and
greedy generation through the engine.  Each test makes its own small configuration and weights."""

from __future__ import annotations

import copy
import json
import math
from types import SimpleNamespace

import pytest
import torch

import plain_fubolix as plain

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16

# ---- configurations ---------------------------------------------------------------------------------------------------

YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}  # with base 10000 and 8 pairs: kept, blended and slowed pairs


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def windowed(mlp=None, heads=4, kv_heads=2, dim=8, size=7, keep=2, dims=4, base=10000.0, scaling=YARN, scale=None):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(scaling)
    return {"type": "attention", "mlp": mlp, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5,
        "mask": {"size": size, "keep_first": keep}, "rot": rot}}


def tempered(mlp=None, heads=4, kv_heads=2, dim=8, vdim=6, coef=0.5, every=4, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention_2", "mlp": mlp, "mixer": m}


def convolved(mlp=None, heads=4, kv_heads=2, dim=8, vdim=6, conv=3, dims=4, base=500.0, scaling=None, scale=None):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(scaling)
    return {"type": "attention_3", "mlp": mlp, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
        "conv": conv, "rot": rot}}


def config(layers, width=40, vocab=89, eps=1e-5, embed_scale=1.7):
    return {"architecture": "Fubolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "layers": layers}


def full_config(**kw):
    """All three mixers, layers with and without a feed-forward; sizes differ from layer to layer."""
    return config([convolved(dense(56), heads=6, kv_heads=2, dim=12, vdim=10, conv=4, dims=8, scaling=YARN),
                   windowed(dense(24), heads=6, kv_heads=3, dim=16, size=9, keep=3, dims=16),
                   tempered(None, heads=2, kv_heads=2, dim=16, vdim=4, every=5),
                   windowed(None, heads=5, kv_heads=1, dim=6, size=5, keep=0, dims=2, scaling=None),
                   convolved(dense(16), heads=3, kv_heads=1, dim=4, vdim=10, conv=2, dims=0)], **kw)


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Names and shapes from the framework's own list, values from here, bfloat16-representable."""
    from nanospec_b200.weights import build_model

    model, _ = build_model(cfg, None, F32, "cpu")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in sorted(model.weight_specs().items()):
        t = torch.randn(spec.shape, generator=g)
        leaf = name.split(".")[-1]
        if len(spec.shape) == 2 and leaf != "conv":
            t = t * (1.5 / math.sqrt(spec.shape[1]))
        elif leaf == "conv":
            t = 0.6 * t
        elif leaf == "alpha":
            t = 0.7 + 0.1 * t
        elif leaf in ("norm", "norm1"):
            t = 1.0 + 0.2 * t
        elif leaf == "b":
            t = 0.3 * t
        out[name] = t.to(BF16).float()   # (sinks: standard normal)
    return out


def write_folder(folder, cfg, weights):
    from nanospec_b200.weights import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {k: v.to(BF16) for k, v in weights.items()})
    return folder


def make(tmp_path, cfg, seed=0, dtype=F32, blocks=64, page=4, slots=4, weights=None):
    from nanospec_b200 import load_model
    from nanospec_b200.engine.step import ModelRunner

    w = weights if weights is not None else random_weights(cfg, seed)
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


def rounding(cfg, w, ids, want, samples=4):
    """Per position: how far bfloat16 storage of the activations alone moves the plain logits: the largest of the rounding
    itself and of `samples` draws of a relative error of that size on every stored activation."""
    worst = distance(plain.forward(cfg, w, ids, rounded=BF16), want)
    for seed in range(samples):
        g = torch.Generator().manual_seed(seed)
        draw = lambda t: t * (1.0 + (torch.rand(t.shape, generator=g, dtype=t.dtype) - 0.5) * 2.0 ** -7)
        worst = torch.maximum(worst, distance(plain.forward(cfg, w, ids, rounded=draw), want))
    return worst


def close(got, want, dtype, what="", noise=None):
    """float32: a few roundings against the logits' spread at every position.  bfloat16: small at the median position, and at
    every position within a few times of what rounding alone does there (`noise`, from `rounding`), never of the size that a
    wrong mask, a lost sink or a wrong page gives elsewhere."""
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

def test_dynamic_tanh_kernel_alone():
    """resid += a + b; out = tanh(alpha * resid) * gain + bias: widths that take the vector form and the scalar one, no branch,
    one and two, all rows and selected rows."""
    from nanospec_b200 import ops

    g = torch.Generator().manual_seed(1)
    for H in (24, 33, 192, 1030, 4096):
        N = 7
        resid, gain, bias = torch.randn(N, H, generator=g) * 2, 1.0 + 0.3 * torch.randn(H, generator=g), torch.randn(H, generator=g)
        alpha = torch.tensor([0.6])
        for dtype in (F32, BF16):
            tol = 2e-6 if dtype == F32 else 8e-3
            a, b = torch.randn(N, H, generator=g).to(dtype), torch.randn(N, H, generator=g).to(dtype)
            for branches in ((), (a,), (a, b)):
                total = resid.double() + sum(x.double() for x in branches)
                want = plain.dynamic_tanh(total, gain.double(), bias.double(), 0.6)
                r = resid.cuda().contiguous()
                out = ops.add_dyt(r, [x.cuda() for x in branches], gain.cuda(), bias.cuda(), alpha.cuda(), torch.empty(N, H, dtype=dtype, device="cuda"))
                assert (out.float().cpu() - want).abs().max() <= tol * float(want.abs().max()), (H, dtype, len(branches))
                assert (r.cpu() - total).abs().max() <= 1e-6 * float(total.abs().max())
                rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32)
                r2 = resid.cuda().contiguous()
                out = ops.add_dyt(r2, [x.cuda() for x in branches], gain.cuda(), bias.cuda(), alpha.cuda(),
                                  torch.empty(4, H, dtype=dtype, device="cuda"), rows=rows.cuda())
                assert (out.float().cpu() - want[rows.long()]).abs().max() <= tol * float(want.abs().max())
                assert torch.equal(r2.cpu(), resid)


def test_squared_relu_kernel_alone():
    from nanospec_b200 import ops

    g = torch.Generator().manual_seed(2)
    for shape in ((5, 24), (3, 7)):
        for dtype in (F32, BF16):
            x = torch.randn(shape, generator=g).to(dtype)
            got = ops.activation(x.cuda(), torch.empty(shape, dtype=dtype, device="cuda"), "relu2")
            want = plain.relu_squared(x.double())
            assert (got.float().cpu() - want).abs().max() <= (1e-6 if dtype == F32 else 1e-2) * float(want.abs().max())


def _paged(k, page, pages, generator):
    """[T, G, d] rows scattered over pages in a shuffled order: ([pages, G, page, d], table [1, blocks])."""
    T, G, d = k.shape
    blocks = -(-T // page)
    order = torch.randperm(pages, generator=generator)[:blocks]
    store = torch.zeros(pages, G, page, d, dtype=k.dtype)
    for t in range(T):
        store[order[t // page], :, t % page] = k[t]
    return store, order.int().view(1, -1)


@pytest.mark.parametrize("d,dv,H,G,window,keep,learned", [(64, 64, 8, 2, 80, 5, False), (128, 128, 4, 4, 0, 0, True), (32, 80, 6, 1, 0, 0, False),
                                                           (16, 16, 2, 2, 33, 0, True), (48, 48, 3, 3, 200, 17, False), (24, 72, 4, 2, 0, 0, True),
                                                           (20, 12, 4, 2, 40, 3, True)])
def test_attention_kernels_with_a_sink_and_gated_heads(d, dv, H, G, window, keep, learned):
    """The exact kernel (both precisions) and the two tensor-core kernels (a prompt's portion on top of cached keys, single
    tokens with one split and with many) against a plain softmax with the sink in its denominator and the heads' gates, over a
    window that keeps the first keys.  The sink counts: the same rows without it differ by far more than the tolerance."""
    from nanospec_b200 import ops
    from nanospec_b200.parts.context import Workspace

    g = torch.Generator().manual_seed(d + H)
    T, page, pages = 333, 16, 40
    scale = d ** -0.5
    q = torch.randn(T, H, d, generator=g).to(BF16).float()
    k = torch.randn(T, G, d, generator=g).to(BF16).float()
    v = torch.randn(T, G, dv, generator=g).to(BF16).float()
    sink = (torch.randn(H, generator=g).abs() + 1.0) if learned else torch.zeros(H)
    gate = torch.randn(T, H + 3, generator=g).to(BF16).float()  # the heads' gates are columns 2 .. 2 + H of wider rows
    mask = plain.window_mask(T, window, keep) if window else plain.causal_mask(T)
    s = torch.einsum("ihd,jhd->hij", q.double(), k.double().repeat_interleave(H // G, 1)) * scale
    vv = v.double().repeat_interleave(H // G, 1)
    p = plain.softmax_with_sink(s, mask, sink.double())
    want = (torch.einsum("hij,jhe->ihe", p, vv) * torch.sigmoid(gate[:, 2: 2 + H].double())[:, :, None]).reshape(T, H * dv)
    plain.SINK = False
    try:
        bare = (torch.einsum("hij,jhe->ihe", plain.softmax_with_sink(s, mask, sink.double()), vv) *
                torch.sigmoid(gate[:, 2: 2 + H].double())[:, :, None]).reshape(T, H * dv)
    finally:
        plain.SINK = True
    assert (bare - want).abs().max() > 0.2
    for dtype in (F32, BF16):
        g2 = torch.Generator().manual_seed(d + H + 1)
        ks, table = _paged(k.to(dtype), page, pages, g2)
        g2 = torch.Generator().manual_seed(d + H + 1)
        vs, _ = _paged(v.to(dtype), page, pages, g2)
        ks, vs, table = ks.cuda(), vs.cuda(), table.cuda()
        qd = q.reshape(T, H * d).to(dtype).cuda()
        gd = gate.to(dtype).cuda()[:, 2: 2 + H]
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        req = torch.zeros(T, dtype=torch.int32, device="cuda")
        out = torch.zeros(T, H * dv, dtype=dtype, device="cuda")
        ops.attention_generic(qd, ks, vs, table, req, pos, out, H, G, d, page, scale, window=window, keep_first=keep, v_dim=dv,
                              sink=sink.cuda(), gate=gd)
        tol = 2e-5 if dtype == F32 else 0.03
        assert (out.float().cpu() - want).abs().max() <= tol * float(want.abs().max()), ("exact", dtype)
    if d % 8 or dv % 8:
        return
    lane = SimpleNamespace(k=ks, v=vs, block_table=table, page_size=page)
    for start, n in ((0, T), (100, 200), (window - 1 if window else 5, 130)):
        tiles = torch.tensor([[0, off] for off in range(0, n, ops.TILE_Q)], dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(positions=pos[start: start + n].contiguous(), qo_indptr=torch.tensor([0, n], dtype=torch.int32, device="cuda"))
        out = torch.zeros(n, H * dv, dtype=BF16, device="cuda")
        ops.attention_prefill(qd[start: start + n].contiguous(), lane, ctx, out, H, G, d, scale, window, tiles, None, keep_first=keep,
                              wide_weights=True, v_dim=dv, sink=sink.cuda(), gate=gd[start: start + n])
        torch.cuda.synchronize()
        assert (out.float().cpu() - want[start: start + n]).abs().max() <= 0.03 * float(want.abs().max()), ("prefill", start, n)
    rows = [0, 1, T - 1, 77, 200] + ([c for c in (window - 1, window, window + 1, window + keep, 2 * window) if 0 < c < T] if window else [])
    for longest in (None, 64):
        B = len(rows)
        ctx = SimpleNamespace(positions=torch.tensor(rows, dtype=torch.int32, device="cuda"), token_req=torch.arange(B, dtype=torch.int32, device="cuda"),
                              qo_indptr=torch.arange(B + 1, dtype=torch.int32, device="cuda"), workspace=Workspace(torch.device("cuda")))
        lane_b = SimpleNamespace(k=ks, v=vs, block_table=table.repeat(B, 1).contiguous(), page_size=page)
        out = torch.zeros(B, H * dv, dtype=BF16, device="cuda")
        ops.attention_decode(qd[rows].contiguous(), lane_b, ctx, out, H, G, d, scale, window, None, B, longest, keep_first=keep,
                             wide_weights=True, v_dim=dv, sink=sink.cuda(), gate=gd[rows].contiguous())
        torch.cuda.synchronize()
        assert (out.float().cpu() - want[rows]).abs().max() <= 0.03 * float(want.abs().max()), ("decode", longest)


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,dv_other,rot_dims", [(3, 2, 12, 8, 8), (3, 2, 16, 8, 16), (5, 1, 48, 24, 32), (2, 2, 64, 64, 16)],
                         ids=["one feature at a time", "eight at a time", "heads of 48", "heads of 64"])
def test_head_preparation_kernel_alone(nq, nkv, d, dv_other, rot_dims, dtype):
    """The convolution with its tail carried from step to step, the head norms before and after the rotation, both pairings, the
    query temperature, keys that double as values, and what lands in the cache: two requests in portions against the plain
    functions over the whole sequences."""
    from nanospec_b200 import ops

    g = torch.Generator().manual_seed(11)
    page = 4
    lengths, cuts = [19, 11], [[5, 1, 2, 11], [2, 6, 1, 2]]
    for case in ("conv", "norm after, values from keys", "norm before, temperature", "one tap"):
        dv = d if case.startswith("norm after") else dv_other
        v_from_k = case.startswith("norm after")
        cols = (nq + nkv) * d + (0 if v_from_k else nkv * dv)
        taps_n = {"conv": 4, "one tap": 1}.get(case, 0)
        taps = (torch.randn(cols, taps_n, generator=g) * 0.6).to(BF16).float() if taps_n else None
        rot = {"dims": rot_dims, "base": 300.0, "scaling": YARN}
        layout = "half" if case == "conv" else "interleaved"
        f, mag = plain.yarn_frequencies(rot)
        gains = (1.0 + 0.3 * torch.randn(2, d, generator=g)) if case.startswith("norm before") else None
        seqs = [torch.randn(n, cols + 8, generator=g).to(dtype).float() for n in lengths]  # the rows are wider than [q | k | v]
        want = []
        for x in seqs:
            u = x[:, :cols].double()
            if taps is not None:
                u = plain.causal_convolution(u, taps.double())
            T = u.shape[0]
            pos = torch.arange(T)
            qh, kh = u[:, : nq * d].view(T, nq, d), u[:, nq * d: (nq + nkv) * d].view(T, nkv, d)
            vals = kh.clone() if v_from_k else u[:, (nq + nkv) * d:].view(T, nkv, dv)
            if gains is not None:
                qh, kh = plain.unit_rms(qh, 1e-5) * gains[0].double(), plain.unit_rms(kh, 1e-5) * gains[1].double()
            qh, kh = plain.rotate(qh, pos, rot, layout), plain.rotate(kh, pos, rot, layout)
            if v_from_k:
                qh, kh = plain.unit_rms(qh, 1e-5), plain.unit_rms(kh, 1e-5)
            if gains is not None:
                qh = qh * (1.0 + 0.4 * torch.log(torch.floor((pos.double() + 1.0) / 3.0) + 1.0))[:, None, None]
            want.append((qh, kh, vals))
        n_pages = 16
        kc = torch.zeros(n_pages, nkv, page, d, dtype=dtype, device="cuda")
        vc = torch.zeros(n_pages, nkv, page, dv, dtype=dtype, device="cuda")
        table = torch.tensor([[3, 9, 1, 12, 7, 0, 0, 0], [5, 2, 14, 0, 0, 0, 0, 0]], dtype=torch.int32, device="cuda")
        state = torch.zeros(3, max(1, (taps_n - 1) * cols) if taps_n else 1, dtype=F32, device="cuda")
        lane = SimpleNamespace(k=kc, v=vc, block_table=table, page_size=page, state=state)
        at, got_q, got_k = [0, 0], [[], []], [[], []]
        for step in range(4):
            ns = [cuts[b][step] for b in range(2)]
            rows = torch.cat([seqs[b][at[b]: at[b] + ns[b]] for b in range(2)]).to(dtype).cuda()
            ctx = SimpleNamespace(
                positions=torch.tensor([at[b] + i for b in range(2) for i in range(ns[b])], dtype=torch.int32, device="cuda"),
                token_req=torch.tensor([b for b in range(2) for _ in range(ns[b])], dtype=torch.int32, device="cuda"),
                qo_indptr=torch.tensor([0, ns[0], ns[0] + ns[1]], dtype=torch.int32, device="cuda"),
                state_slot=torch.tensor([1, 0], dtype=torch.int32, device="cuda"), n_requests=2)
            out = torch.zeros_like(rows) if taps_n > 1 else rows
            ops.head_prepare_store(rows, out, ctx, lane, nq, nkv, d, dv, inv_freq=f.float().cuda(), magnitude=mag, interleaved=layout == "interleaved",
                                   norm="after" if v_from_k else "before" if gains is not None else None,
                                   q_gain=gains[0].cuda() if gains is not None else None, k_gain=gains[1].cuda() if gains is not None else None,
                                   eps=1e-5, q_temp=(0.4, 3.0) if gains is not None else None, taps=taps.t().contiguous().cuda() if taps is not None else None,
                                   v_from_k=v_from_k)
            o = out.float().cpu()
            row = 0
            for b in range(2):
                got_q[b].append(o[row: row + ns[b], : nq * d])
                got_k[b].append(o[row: row + ns[b], nq * d: (nq + nkv) * d])
                row += ns[b]
                at[b] += ns[b]
        tol = 3e-6 if dtype == F32 else 1.2e-2
        for b in range(2):
            qh, kh, vals = want[b]
            T = lengths[b]
            size = float(qh.abs().max())
            assert (torch.cat(got_q[b]).double() - qh.reshape(T, -1)).abs().max() <= tol * size, (case, "q", b)
            assert (torch.cat(got_k[b]).double() - kh.reshape(T, -1)).abs().max() <= tol * size, (case, "k", b)
            for t in range(T):
                pg = int(table[b, t // page])
                assert (kc[pg, :, t % page].float().cpu().double() - kh[t]).abs().max() <= tol * size, (case, "cached k", b, t)
                assert (vc[pg, :, t % page].float().cpu().double() - vals[t]).abs().max() <= tol * float(vals.abs().max()), (case, "cached v", b, t)


# ---- each mechanism alone -----------------------------------------------------------------------------------------------

SINGLE = {
    "windowed attention alone": lambda: config([windowed()]),
    "a window of one, no kept keys": lambda: config([windowed(size=1, keep=0, heads=2, kv_heads=1)]),
    "more kept keys than the window holds": lambda: config([windowed(size=3, keep=6)]),
    "every query head with keys of its own, whole heads turn, plain frequencies": lambda: config([windowed(heads=3, kv_heads=3, dims=8, scaling=None, base=300.0)]),
    "five query heads to a key head, nothing turns": lambda: config([windowed(heads=5, kv_heads=1, dim=6, dims=0, size=11)]),
    "tempered attention alone": lambda: config([tempered()]),
    "tempered attention without a temperature, one head, values wider than keys": lambda: config([tempered(heads=1, kv_heads=1, dim=4, vdim=18, every=0)]),
    "a temperature that grows with every token": lambda: config([tempered(every=1, coef=1.1, heads=6, kv_heads=2)]),
    "convolved attention alone": lambda: config([convolved()]),
    "one tap": lambda: config([convolved(conv=1, heads=2, kv_heads=2)]),
    "two taps, whole heads turn with scaled frequencies": lambda: config([convolved(conv=2, dim=8, dims=8, scaling=YARN, base=10000.0)]),
    "six taps, three query heads to a key head": lambda: config([convolved(conv=6, heads=6, kv_heads=2, dim=10, vdim=14, dims=6)]),
    "feed-forward beside the mixer": lambda: config([tempered(dense(24))]),
    "two layers: the pending pair reaches the next norm": lambda: config([windowed(dense(16)), convolved(dense(32))]),
    "an embedding that is not scaled": lambda: config([windowed(dense(16))], embed_scale=1.0),
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


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
def test_sublayers_with_products_of_their_own(dtype, tmp_path):
    """The arrangement with its packing switched off: four products a layer, the pair of branches pending for the next norm."""
    from nanospec_b200.parts.block import ParallelBlock

    cfg = config([windowed(dense(16), heads=4, kv_heads=2, dim=16), convolved(dense(32), dim=16, vdim=8), tempered(dense(24), dim=16, vdim=16)])
    ids = tokens(37, cfg["vocab"], 5)
    ParallelBlock.PACK = False
    try:
        runner, w = make(tmp_path, cfg, seed=77, dtype=dtype)
    finally:
        ParallelBlock.PACK = True
    assert all(b.w_in is None for b in runner.model.blocks)
    packed, _ = make(tmp_path / "p", cfg, seed=77, dtype=dtype, weights=w)
    assert all(b.w_in is not None for b in packed.model.blocks)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want)
    for cuts in ([37], [], [2, 3, 2, 11, 5, 2]):
        close(run_cut(runner, 0, ids, cuts), want, dtype, f"own products, portions {cuts or 'of one'}", noise)
        close(run_cut(packed, 0, ids, cuts), want, dtype, f"packed products, portions {cuts or 'of one'}", noise)


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_the_next_norm_in_the_output_product(graphs, tmp_path):
    """bfloat16, a width in multiples of 128, steps of up to 64 tokens: the packed output product adds its result to the stream and
    applies the next layer's norm in its epilogue.  Portions of every size beside it, and generation through the engine."""
    from nanospec_b200 import Engine, EngineConfig, SamplingParams
    from nanospec_b200.ops import lib

    cfg = config([windowed(dense(128), heads=4, kv_heads=2, dim=16), convolved(dense(64), dim=16, vdim=8), tempered(dense(128), dim=32, vdim=16),
                  windowed(None, heads=2, kv_heads=1, dim=32, size=20), tempered(dense(64), dim=16, vdim=16)], width=128)
    runner, w = make(tmp_path, cfg, seed=91, dtype=BF16, page=16, blocks=40)
    ids = tokens(150, cfg["vocab"], 6)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want, samples=2)
    lib.start_kernel_timing()
    got = run_cut(runner, 0, ids, [64, 2, 30, 3])
    seen = lib.stop_kernel_timing()
    assert seen.get("ns_gemm_bf16_tc_dyt", (0, 0.0))[0] > 0, sorted(seen)
    close(got, want, BF16, "the norm in the product's epilogue", noise)
    close(run_cut(runner, 1, ids, [150]), want, BF16, "the same model, a whole prompt", noise)
    eng = Engine(runner.model, EngineConfig(num_blocks=64, block_size=16, max_running=3, prefill_chunk=40, cuda_graphs=graphs, graph_buckets=(1, 2, 4)))
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (3, 70, 1, 17)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    for p, out in zip(prompts, outs):
        z = plain.forward(cfg, w, p + out)
        for j, tok in enumerate(out):
            row = z[len(p) + j - 1]
            assert float(row.max() - row[tok]) / float(z.std()) <= 0.1, f"token {j}"


@pytest.mark.parametrize("width", [36, 128], ids=["own products", "packed products"])
def test_weights_replaced_in_place(width, tmp_path):
    """`update_weights` on a bound model: the sublayers hold views of the block's packed matrices, and new tensors land there."""
    from nanospec_b200.weights import update_weights

    cfg = config([convolved(dense(64), dim=16, vdim=8), windowed(dense(32), heads=4, kv_heads=2, dim=16), tempered(None, dim=16, vdim=16)], width=width)
    runner, w = make(tmp_path, cfg, seed=5)
    assert (runner.model.blocks[0].w_in is not None) == (width == 128)
    ids = tokens(40, cfg["vocab"], 9)
    close(run_cut(runner, 0, ids, [17, 2]), plain.forward(cfg, w, ids), F32, "before")
    w2 = random_weights(cfg, 6)
    update_weights(runner.model, {k: v.clone() for k, v in w2.items()})
    got = run_cut(runner, 1, ids, [17, 2])
    close(got, plain.forward(cfg, w2, ids), F32, "after")
    assert float(distance(got, plain.forward(cfg, w, ids)).max()) > 0.1


@pytest.mark.parametrize("packed", [False, True], ids=["own products", "packed products"])
def test_float32_logits_do_not_depend_on_the_cut(packed, tmp_path):
    """In float32 every sum runs in an order fixed per output element: whole, token by token and in portions give the same bits."""
    cfg = config([windowed(dense(128), heads=4, kv_heads=2, dim=16), convolved(dense(64), dim=16, vdim=8), tempered(dense(128), dim=32, vdim=16)],
                 width=128) if packed else full_config()
    runner, _ = make(tmp_path, cfg, seed=3, page=4, blocks=80)
    assert (runner.model.blocks[0].w_in is not None) == packed
    ids = tokens(150, cfg["vocab"], 5)
    whole = run_cut(runner, 0, ids, [150])
    for i, cuts in enumerate(([], [2, 3, 2, 11, 5, 2], [64, 65, 1, 1, 17])):
        assert torch.equal(run_cut(runner, i + 1, ids, cuts), whole), cuts


def test_layers_one_by_one(tmp_path):
    """The stream after every layer, in float32, against the plain statement's."""
    from nanospec_b200.engine.step import StepEntry

    cfg = full_config()
    runner, w = make(tmp_path, cfg, seed=3)
    ids = tokens(29, cfg["vocab"], 8)
    want, single = [], []
    plain.forward(cfg, w, ids, layers_out=want)
    plain.F = F32  # the same statement in float32: what 32-bit rounding alone does to each layer's stream
    try:
        plain.forward(cfg, w, ids, layers_out=single)
    finally:
        plain.F = torch.float64
    got = []

    def probe(i, resid, pending):
        x = resid.detach().cpu().double().clone()
        for p in pending if isinstance(pending, (tuple, list)) else (pending,):
            if p is not None:
                x += p.detach().cpu().double()
        got.append(x)

    runner.begin(0)
    ctx, rows, _ = runner.build_context([StepEntry(0, ids, [])])
    ctx.extras["probe"] = probe
    runner.forward(ctx, rows)
    runner.end(0)
    assert len(got) == len(want)
    for i, (a, b, c) in enumerate(zip(got, want, single)):
        limit = max(1e-5 * float(b.abs().max()), 3 * float((c.double() - b).abs().max()))
        assert (a - b).abs().max() <= limit, f"layer {i}: {float((a - b).abs().max())} (limit {limit})"


# ---- window edges, kept first keys, the sink, the gate, the temperature, the convolution --------------------------------------

def window_edge_case(dim):
    """Windowed attention first, then the two other mixers.  In the first layer the norm is made the bare tanh, every query head's map
    is its key head's with the halves of its input swapped, and four tokens B have the embeddings of four tokens A with the halves
    swapped: a B's query points where its A's key points (the heads are of unit length, so a score cannot be scaled up, but it can be
    made the largest there is).  The pairs sit just inside the window (8 back of 9), just outside it (9 back), on the last kept
    position and on the first that is not kept."""
    size, keep, width = 9, 3, 40
    cfg = config([windowed(dense(16), heads=4, kv_heads=2, dim=dim, size=size, keep=keep, dims=4, scale=1.5),
                  tempered(None, heads=4, kv_heads=2, dim=dim, vdim=dim, every=7, coef=2.5, scale=1.0),
                  convolved(None, heads=4, kv_heads=2, dim=dim, vdim=dim, conv=3, dims=dim, scale=0.9)], width=width)
    w = random_weights(cfg, 14)
    w["l0.norm1"], w["l0.norm1.b"] = torch.ones(width), torch.zeros(width)
    w["l0.mix.q"] = torch.roll(w["l0.mix.k"], width // 2, dims=1).view(2, 1, dim, width).expand(2, 2, dim, width).reshape(4 * dim, width).clone()
    for i in range(4):
        w["embed"][84 + i] = torch.roll(w["embed"][80 + i], width // 2)
    ids = [t % 80 for t in tokens(45, cfg["vocab"], 17)]
    ids[keep - 1], ids[30] = 80, 84        # seen only because it is kept
    ids[keep], ids[31] = 81, 85            # the first that is not kept
    ids[12], ids[12 + size - 1] = 82, 86   # the window's last key
    ids[14], ids[14 + size] = 83, 87       # one beyond it
    return cfg, w, ids, size, keep


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [8, 16], ids=["exact", "tensor-core"])
def test_window_edges_kept_keys_and_the_other_constants(dim, dtype, tmp_path):
    """A window one key longer or shorter, one kept key more or fewer, a softmax without its sink, gates left out, another
    temperature step, a lost tap or a lost gain move the plain logits by far more than the engine differs from the right ones - in a
    prompt, in portions that cut through windows and pages, and token by token.  Heads of 8 run in the exact kernel in both types,
    heads of 16 in the tensor-core kernels in bfloat16."""
    cfg, w, ids, size, keep = window_edge_case(dim)
    runner, w = make(tmp_path, cfg, seed=14, dtype=dtype, page=4, weights=w)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want)
    calm = noise <= 0.05  # bfloat16: the variants are told apart at the positions that rounding leaves alone
    wrong = window_edge_variants(cfg, w, ids, size, keep)
    for cuts in ([45], [], [size - 1, 2, size, 3, 2, 2, size + 1], [4, 4, 4, 4, 4], [size, size, size]):
        got = run_cut(runner, 0, ids, cuts)
        close(got, want, dtype, f"window edges, portions {cuts or 'of one'}", noise)
        keepers = torch.ones_like(calm) if dtype == F32 else calm
        right = float(distance(got, want)[keepers].max())
        for i, z in enumerate(wrong):
            off = float(distance(got, z)[keepers].max())
            assert off > (10 if dtype == F32 else 3) * right and off > 0.03, f"variant {i} is not told apart: {off} against {right}"


def window_edge_variants(cfg, w, ids, size, keep):
    wrong = []
    for key, base in (("size", size), ("keep_first", keep)):
        for delta in (-1, 1):
            other = copy.deepcopy(cfg)
            other["layers"][0]["mixer"]["mask"][key] = base + delta
            wrong.append(plain.forward(other, w, ids))
    for every in (6, 8):
        other = copy.deepcopy(cfg)
        other["layers"][1]["mixer"]["q_temp"]["every"] = every
        wrong.append(plain.forward(other, w, ids))
    plain.SINK = False
    try:
        wrong.append(plain.forward(cfg, w, ids))
    finally:
        plain.SINK = True
    for name, value in (("l0.mix.g", 0.0), ("l2.mix.sink", -30.0), ("l1.mix.k.norm", 1.0)):
        lost = dict(w)
        lost[name] = torch.full_like(w[name], value)
        wrong.append(plain.forward(cfg, lost, ids))
    lost = dict(w)
    lost["l2.mix.k.conv"] = w["l2.mix.k.conv"].clone()
    lost["l2.mix.k.conv"][:, 0] = 0.0   # the tap that reaches two tokens back
    wrong.append(plain.forward(cfg, lost, ids))
    return wrong


def far_key_case():
    """One layer of tempered attention (every earlier key) whose last token looks for one token far back.  The layer's norm is made
    the bare tanh, the queries' map is the keys' with the halves of its input swapped, and token 49's embedding is token 48's with
    its halves swapped: 49's query points where 48's key points, so the last position (a 49) puts its weight on the only 48."""
    width = 64
    cfg = config([tempered(heads=2, kv_heads=2, dim=32, vdim=8, every=50, coef=0.2, scale=1.4)], width=width, vocab=50)
    w = random_weights(cfg, 41)
    w["l0.norm1"], w["l0.norm1.b"] = torch.ones(width), torch.zeros(width)
    w["l0.mix.q.norm"], w["l0.mix.k.norm"] = torch.ones(32), torch.ones(32)
    w["l0.mix.q"] = torch.roll(w["l0.mix.k"], width // 2, dims=1).clone()
    w["embed"][49] = torch.roll(w["embed"][48], width // 2)
    ids = tokens(450, 48, 42)
    ids[31], ids[-1] = 48, 49          # 48 occurs nowhere else; position 31 is the last of the second page of 16
    lost = list(ids)
    lost[31] = 47
    return cfg, w, ids, lost


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
def test_a_key_far_back(dtype, tmp_path):
    """The last token's query looks for one token 418 positions back, and a model that had lost that key would answer otherwise -
    in a whole prompt, as a decoded token and in portions."""
    cfg, w, ids, lost = far_key_case()
    runner, w = make(tmp_path, cfg, seed=41, dtype=dtype, page=16, blocks=40, weights=w)
    want = plain.forward(cfg, w, ids)
    assert float(distance(plain.forward(cfg, w, lost)[-1:], want[-1:]).max()) > 0.5
    for cuts in ([450], [449], [200, 100, 2, 140]):
        got = run_cut(runner, 0, ids, cuts)
        assert float(distance(got[-1:], want[-1:]).max()) <= (2e-4 if dtype == F32 else 0.1), cuts


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
def test_kept_keys_far_behind_the_window(dtype, tmp_path):
    """Two hundred positions on, in decoding and in portions, the kept first keys are still read from their pages (which were never
    given back) at their own positions, and the keys between them and the window are not."""
    cfg = config([windowed(dense(16), heads=4, kv_heads=2, dim=16, size=21, keep=5, dims=8, scale=1.5)])
    runner, w = make(tmp_path, cfg, seed=52, dtype=dtype, page=4, blocks=60)
    ids = tokens(230, cfg["vocab"], 53)
    want = plain.forward(cfg, w, ids)
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["mask"]["keep_first"] = 4
    assert float(distance(plain.forward(other, w, ids)[200:], want[200:]).max()) > 0.05
    noise = rounding(cfg, w, ids, want, samples=1) if dtype == BF16 else None
    for cuts in ([230], [30], [100, 2, 61, 40, 3]):
        close(run_cut(runner, 0, ids, cuts), want, dtype, f"kept keys, portions {cuts}", noise)


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
    runner, w = make(tmp_path, cfg, seed=23, blocks=48, page=4)
    ids = tokens(150, cfg["vocab"], 24)
    close(run_cut(runner, 0, ids, [5]), plain.forward(cfg, w, ids), F32, "long decoding")


# ---- batches, pages and slots that are used again ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [F32, BF16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [31, 32])
def test_unequal_batches_and_reuse(seed, dtype, tmp_path):
    """Up to four requests of unequal lengths side by side, portions of some beside single tokens of others, on a pool
    that only their peak fits and four state slots, requests ending and new ones taking their pages and slots: every position
    as alone."""
    from nanospec_b200.engine.step import StepEntry

    cfg = full_config()
    runner, w = make(tmp_path, cfg, seed=seed, dtype=dtype, blocks=30, page=4, slots=4)
    g = torch.Generator().manual_seed(seed)
    lengths = [23, 5, 41, 2, 17, 30, 9, 1, 12]
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

@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_from_seeds(seed, tmp_path):
    g = torch.Generator().manual_seed(3000 + seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    layers = []
    for _ in range(pick([1, 2, 3, 5])):
        mlp = pick([None, dense(pick([8, 20, 64]))])
        kind = pick(["windowed", "tempered", "convolved"])
        kv = pick([1, 2, 3])
        heads = kv * pick([1, 2, 4])
        dim = pick([2, 8, 12, 16, 32])
        scale = pick([None, 0.6, 0.11])
        if kind == "windowed":
            layers.append(windowed(mlp, heads=heads, kv_heads=kv, dim=dim, size=pick([1, 3, 8, 33, 100]), keep=pick([0, 1, 4, 9]),
                                   dims=pick([0, 2, dim]), base=pick([100.0, 50000.0]), scaling=pick([None, YARN]), scale=scale))
        elif kind == "tempered":
            layers.append(tempered(mlp, heads=heads, kv_heads=kv, dim=dim, vdim=pick([2, 8, 20, dim]), coef=pick([0.1, 0.9]),
                                   every=pick([0, 1, 6, 64]), scale=scale))
        else:
            layers.append(convolved(mlp, heads=heads, kv_heads=kv, dim=dim, vdim=pick([2, 8, 20, dim]), conv=pick([1, 2, 4, 5]),
                                    dims=pick([0, 2, dim]), base=pick([100.0, 50000.0]), scaling=pick([None, YARN]), scale=scale))
    cfg = config(layers, width=pick([16, 24, 72, 33]), vocab=pick([50, 131]), eps=pick([1e-5, 1e-6, 1e-3]), embed_scale=pick([1.0, 0.5, 4.0]))
    for dtype in (F32, BF16):
        runner, w = make(tmp_path, cfg, seed=seed, dtype=dtype, page=pick([2, 4, 16]))
        ids = tokens(48, cfg["vocab"], seed)
        want = plain.forward(cfg, w, ids)
        noise = rounding(cfg, w, ids, want)
        for cuts in ([48], [7, 2, 2, 19, 3], []):
            close(run_cut(runner, 0, ids, cuts), want, dtype, f"seed {seed}, portions {cuts or 'of one'}: {json.dumps(cfg)[:300]}", noise)


@pytest.mark.parametrize("dim,vdim,heads,kv_heads,size", [(64, 32, 8, 2, 88), (128, 128, 4, 4, 70), (32, 64, 6, 1, 130), (16, 16, 4, 2, 40), (48, 24, 2, 1, 75)])
def test_tensor_core_sizes(dim, vdim, heads, kv_heads, size, tmp_path):
    """Head sizes that the tensor-core attention kernels take (values as wide as keys, narrower, wider), in bfloat16, over prompts
    long enough for several key tiles and windows, with portions and single tokens; float32 beside it."""
    cfg = config([windowed(dense(64), heads=heads, kv_heads=kv_heads, dim=dim, size=size, keep=6, dims=dim // 2),
                  tempered(None, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, every=32),
                  convolved(None, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=4, dims=dim // 2, scaling=YARN)], width=64)
    ids = tokens(300, cfg["vocab"], size)
    w = random_weights(cfg, size)
    want = plain.forward(cfg, w, ids)
    noise = rounding(cfg, w, ids, want, samples=2)
    for dtype in (BF16, F32):
        runner, _ = make(tmp_path, cfg, seed=size, dtype=dtype, blocks=80, page=16, weights=w)
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
