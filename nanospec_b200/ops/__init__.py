"""Python faces of the CUDA kernels.  Each function checks its tensors (device, dtype,
layout) and launches on the current CUDA stream; none of them has a CPU or library path
except `linear` in bfloat16, which may hand a plain matrix product to cuBLAS.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import lib
from .lib import KernelError

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dt}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)  # the handle without a Stream object around it


def _stream() -> int:
    """The current CUDA stream of the current device, as the integer that the C ABI takes (asked for
    at every launch, so that stream contexts and graph captures are followed)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must live on a CUDA device; there is no CPU path")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _i32(t: torch.Tensor | None, name: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n] = float(table[ids[n]]); out is the fp32 residual stream [N, hidden]."""
    _cuda(table, ids, out)
    _i32(ids, "ids")
    n, hidden = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: out must be contiguous float32 and the table contiguous")
    if table.shape[1] != hidden or ids.numel() != n:
        raise KernelError(f"embed: table {tuple(table.shape)}, ids {ids.numel()}, out {tuple(out.shape)} do not agree")
    lib.call("ns_embed", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, hidden, table.shape[0],
             dtype_code(table.dtype), _stream())
    return out


def take_ids(ids: torch.Tensor, dst_rows: torch.Tensor, src: torch.Tensor, src_rows: torch.Tensor) -> None:
    """ids[dst_rows[i]] = src[src_rows[i]]: a step takes, on the device, the tokens that the step before it sampled."""
    _cuda(ids, dst_rows, src, src_rows)
    for t, name in ((ids, "ids"), (dst_rows, "dst_rows"), (src, "src"), (src_rows, "src_rows")):
        _i32(t, name)
    if dst_rows.numel() != src_rows.numel():
        raise KernelError("take_ids: one source row per destination row")
    lib.call("ns_take_ids", ids.data_ptr(), dst_rows.data_ptr(), src.data_ptr(), src_rows.data_ptr(), dst_rows.numel(), _stream())


def add_rmsnorm(resid: torch.Tensor, branch: torch.Tensor | None, gain: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None, write_resid: bool = True) -> torch.Tensor:
    """resid (+= branch); out = rmsnorm(resid) * gain.  With `rows`, output row j reads
    input row rows[j] and the residual is left unchanged."""
    _cuda(resid, branch, gain, out, rows)
    _i32(rows, "rows")
    hidden = resid.shape[1]
    n_rows = out.shape[0]
    if resid.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream and the gain are float32")
    if not (resid.is_contiguous() and out.is_contiguous() and gain.is_contiguous()) or out.shape[1] != hidden \
            or gain.numel() != hidden:
        raise KernelError("add_rmsnorm: operands must be contiguous and agree on the width")
    if branch is not None and (branch.dtype != out.dtype or branch.shape != resid.shape or not branch.is_contiguous()):
        raise KernelError("add_rmsnorm: the branch must match the residual's shape and the output's dtype")
    if rows is None and n_rows != resid.shape[0]:
        raise KernelError("add_rmsnorm: out and resid differ in rows")
    if rows is not None:
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm: one row index per output row")
        write_resid = False
    lib.call("ns_add_rmsnorm", resid.data_ptr(), _ptr(branch), gain.data_ptr(), out.data_ptr(), _ptr(rows), n_rows,
             hidden, float(eps), int(bool(write_resid)), dtype_code(out.dtype), _stream())
    return out


def residual_add(resid: torch.Tensor, branch: torch.Tensor) -> torch.Tensor:
    _cuda(resid, branch)
    if resid.dtype != torch.float32 or resid.shape != branch.shape or not (resid.is_contiguous() and branch.is_contiguous()):
        raise KernelError("residual_add: float32 residual and a branch of the same shape, both contiguous")
    lib.call("ns_residual_add", resid.data_ptr(), branch.data_ptr(), resid.shape[0], resid.shape[1],
             dtype_code(branch.dtype), _stream())
    return resid


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> torch.Tensor:
    """out[n, j] = silu(gate_up[n, j]) * gate_up[n, I + j]; with `block` > 0 gate and up alternate in
    runs of `block` features instead (gate j at (j // block) * 2 * block + j % block, up `block` further)."""
    _cuda(gate_up, out)
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter) or gate_up.dtype != out.dtype or not (gate_up.is_contiguous() and out.is_contiguous()):
        raise KernelError("swiglu: gate_up must be [N, 2I] and out [N, I], same dtype, contiguous")
    lib.call("ns_swiglu", gate_up.data_ptr(), out.data_ptr(), n, inter, int(block), dtype_code(out.dtype), _stream())
    return out


class _TensorCoreGemmState:
    """Per-device state of the tcgen05 matrix product: the flag that a timed-out wait sets."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.error = torch.zeros(1, dtype=torch.int32, device=device)


_tc_state: dict[torch.device, _TensorCoreGemmState] = {}
_sm_counts: dict[int, int] = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200): the one place the launch heuristics
    below take the size of the chip from."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


USE_TENSOR_CORE_GEMM = True  # the hand-written tcgen05 kernel; False hands every bf16 product to cuBLAS
# Products with more tokens than this go to cuBLAS, whose kernels are ahead of the hand-written
# one there (measured in decode steps of the 8B shape with 1,024 tokens of context: with 32 tokens the
# hand-written kernel and its fused epilogues take 3.64 ms against 4.40 ms, with 48 tokens 4.71 ms against
# 4.80 ms, with 64 tokens 4.79 ms against 4.96 ms; at 2,048 tokens it reaches 68-85 % of cuBLAS); None = no limit.
TENSOR_CORE_GEMM_MAX_TOKENS: int | None = 64


def _tc(device: torch.device) -> _TensorCoreGemmState:
    st = _tc_state.get(device)
    if st is None:
        st = _tc_state[device] = _TensorCoreGemmState(device)
    return st


def set_programmatic_launch(enabled: bool) -> None:
    """Kernels may overlap the tail of their predecessor in the stream (default on)."""
    lib.call("ns_set_pdl", int(bool(enabled)))


def check_kernel_errors(device: torch.device | None = None) -> None:
    """Raises if a kernel recorded a timed-out wait since the last check (one small device read)."""
    for dev, st in _tc_state.items():
        if device is not None and dev != device:
            continue
        code = int(st.error.item())
        if code:
            st.error.zero_()
            what = {1: "matrix product: the TMA producer waited for a free stage", 2: "matrix product: the MMA issuer waited for a tile",
                    3: "matrix product: the epilogue waited for the accumulator", 4: "matrix product: copies in flight did not land",
                    11: "prefill attention: the loader waited for a free stage", 12: "prefill attention: the MMA issuer waited",
                    13: "prefill attention: a softmax warp waited", 21: "decode attention: the loader waited for a free stage",
                    22: "decode attention: a warp waited for its keys",
                    31: "wait probe: nobody arrives at its barrier"}.get(code, "?")
            raise KernelError(f"a kernel gave up waiting on an mbarrier (the limit is two seconds) - {what} (code {code}); "
                              "its output is not valid")


def wait_probe(device: torch.device, limit_ns: int = 1_000_000) -> bool:
    """Launches the one-block kernel of csrc/wait_probe.cu, whose only thread waits `limit_ns` on a barrier at
    which nobody arrives, gives up and records its code in the device's error word, as the production kernels'
    bounded waits do.  Returns whether the wait completed (it cannot); `check_kernel_errors` raises afterwards."""
    st = _tc(torch.device(device) if not isinstance(device, torch.device) else device)
    ok = torch.full((1,), -1, dtype=torch.int32, device=st.device)
    lib.call("ns_wait_probe", st.error.data_ptr(), int(limit_ns), ok.data_ptr(), _stream())
    return bool(ok.item() == 1)


def gemm_splits(M: int, N: int, K: int) -> int:
    """How many blocks share the k range of one output tile: enough to occupy the SMs when the
    output has few tiles (a decode step), 1 when it has many."""
    tokens_per_block = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
    tiles = -(-N // 128) * -(-M // tokens_per_block)
    k_blocks = -(-K // 64)
    resident = sm_count() * (2 if tokens_per_block <= 64 else 1)
    # a block keeps at least 8 k blocks of 64, or 4 in steps of up to 16 tokens, whose six stages then hold a block's
    # whole share of a small matrix before the step's predecessor has finished (measured at the 1B shape, 8 requests:
    # 0.865 ms per step against 0.887; at 64 requests the finer split costs 2 %)
    def splits_with(min_k_blocks: int) -> int:
        want = max(1, min(8, resident // tiles, k_blocks // min_k_blocks))
        return 1 << (want.bit_length() - 1)  # the blocks of a tile form a cluster of 1, 2, 4 or 8

    splits = splits_with(4 if M <= 16 else 8)
    if tiles * splits < sm_count():
        # fewer blocks than SMs (the 3B shape's output projection at 64 requests: 24 tiles x 4 blocks): the finer split
        # after all (continuous batching at that shape: 13,290 against 13,200 output tokens / s)
        splits = splits_with(4)
    return splits


def linear_tensor_core(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int | None = None) -> bool:
    """The tcgen05 kernel (csrc/gemm_tcgen05.cu).  Returns False, having done nothing, when the
    operands do not meet TMA's rules (K and the row strides multiples of 8 elements, 16-byte bases)."""
    M, K = x.shape
    N = w.shape[0]
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 \
            or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    st = _tc(x.device)
    if splits is None:
        splits = gemm_splits(M, N, K)
    lib.call("ns_gemm_bf16_tc", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
             out.stride(0), int(out.dtype == torch.float32), splits, st.error.data_ptr(), _stream())
    return True


FUSE_NORM = True  # a decode step's products take over the residual sum and the norm that follows them


@dataclass
class NormSink:
    """Where a product's output goes when the residual sum and the RMSNorm that follow are folded
    into its epilogue: `resid` [N, H] float32 is updated in place, `gain` [H] and `eps` are the norm's."""

    resid: torch.Tensor
    gain: torch.Tensor
    eps: float
    workspace: object  # parts.context.Workspace: the buffers of the result come from it


@dataclass
class RowScaled:
    """Normed activations that still lack the norm's scale: `x` [N, H] = gain * resid in the compute
    dtype and `partials` [N, P] float32, per-row partial sums of resid^2.  Row n's scale is
    rsqrt(sum(partials[n]) / hidden + eps); the product that reads `x` applies it to its output rows
    (a product is linear in a per-row scale of its input).  `gain` identifies the norm it stands for."""

    x: torch.Tensor
    partials: torch.Tensor
    hidden: int
    eps: float
    gain: torch.Tensor

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype


@dataclass
class TanhSink:
    """Where a product's output goes when the residual sum and a norm WITHOUT statistics that follow are folded into its epilogue:
    `resid` [N, H] float32 is updated in place and tanh(alpha * resid) * gain + bias comes back complete, as a `Normed`."""

    resid: torch.Tensor
    gain: torch.Tensor
    bias: torch.Tensor | None
    alpha: torch.Tensor  # one float32 on the device
    workspace: object


@dataclass
class Normed:
    """Normed activations `x` [N, H] in the compute dtype that a product's epilogue has left, the stream already updated;
    `gain` identifies the norm they stand for."""

    x: torch.Tensor
    gain: torch.Tensor


def _tma_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[1]
    return not (K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.stride(1) != 1 or w.stride(1) != 1
                or x.data_ptr() % 16 or w.data_ptr() % 16)


def norm_fusion_ok(n_tokens: int, dtype: torch.dtype, *weights: torch.Tensor) -> bool:
    """Whether a step of `n_tokens` in `dtype` may hand normed activations on as `RowScaled` to products
    with these weights (and fold a norm into a product with them): the tcgen05 kernel with a tile of up to 64
    tokens, feature counts in multiples of 128, rows that TMA can address."""
    if not (FUSE_NORM and USE_TENSOR_CORE_GEMM and dtype == torch.bfloat16 and 0 < n_tokens <= 64):
        return False
    if TENSOR_CORE_GEMM_MAX_TOKENS is not None and n_tokens > TENSOR_CORE_GEMM_MAX_TOKENS:
        return False
    return all(w.dtype == torch.bfloat16 and w.shape[0] % 128 == 0 and w.shape[1] % 8 == 0 and w.stride(1) == 1
               and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 for w in weights)


def _linear_norm(x, w: torch.Tensor, out: torch.Tensor | None, gated: bool, sink: NormSink | None):
    """The tcgen05 product with the norm epilogues: x a tensor or RowScaled; returns `out`, or the
    RowScaled that the sink produced."""
    scaled = x if isinstance(x, RowScaled) else None
    xt = scaled.x if scaled is not None else x
    M, K = xt.shape
    N = w.shape[0]
    if w.shape[1] != K or not _tma_ok(xt, w) or M > 64:
        raise KernelError(f"linear: the norm epilogues cannot take x {tuple(xt.shape)}, w {tuple(w.shape)}")
    splits = gemm_splits(M, N, K)
    res = None
    if sink is not None:
        if gated or N % 128 or sink.resid.shape != (M, N) or not sink.resid.is_contiguous():
            raise KernelError("linear: a norm sink takes an ungated product whose width is the residual's, a multiple of 128")
        ws = sink.workspace
        res = RowScaled(ws.get("sink_x", M, N, torch.bfloat16), ws.get("sink_partials", M, (N // 128) * splits, torch.float32),
                        N, sink.eps, sink.gain)
    elif out is None or out.shape != (M, N // 2 if gated else N) or out.stride(1) != 1:
        raise KernelError("linear: the output does not fit the product")
    lib.call("ns_gemm_bf16_tc_norm", xt.data_ptr(), w.data_ptr(), _ptr(out), M, N, K, xt.stride(0), w.stride(0),
             out.stride(0) if out is not None else 0, int(out is not None and out.dtype == torch.float32), splits, int(gated),
             _ptr(scaled.partials if scaled is not None else None), scaled.partials.shape[1] if scaled is not None else 0,
             scaled.hidden if scaled is not None else 0, float(scaled.eps) if scaled is not None else 0.0,
             _ptr(sink.resid if sink is not None else None), _ptr(sink.gain if sink is not None else None),
             _ptr(res.x if res is not None else None), _ptr(res.partials if res is not None else None),
             N if sink is not None else 0, _tc(xt.device).error.data_ptr(), _stream())
    return res if res is not None else out


def linear(x, w: torch.Tensor, out: torch.Tensor, sink: NormSink | None = None):
    """out[M, N] = x[M, K] @ w[N, K]^T with fp32 accumulation.

    `x` may be a `RowScaled` (its rows' scale is applied to the output).  With a `sink` that the product
    can fold in (`norm_fusion_ok`), nothing is written to `out`: the residual is updated and a `RowScaled`
    for the norm that follows is returned; otherwise `out` is returned and the caller runs the norm.  A `TanhSink` (a norm
    without statistics follows) likewise: the stream is updated and a `Normed` returned, or `out`.

    float32: the CUDA-core kernel (true fp32, k-ascending sums, independent of M).
    bfloat16: the tcgen05 kernel; operands that TMA cannot address (K or a row stride that is no
    multiple of 8) are a plain matrix product for cuBLAS, as the reference hands its `nn.Linear`
    calls to it (model/llama.py:175,184,195).  `out` may be bfloat16 or float32.
    """
    if isinstance(sink, TanhSink):
        if norm_fusion_ok(x.shape[0], x.dtype, w) and sink.resid.shape == (x.shape[0], w.shape[0]) and sink.resid.is_contiguous() \
                and _tma_ok(x, w):
            M, K = x.shape
            N = w.shape[0]
            normed = sink.workspace.get("sink_x", M, N, torch.bfloat16)
            lib.call("ns_gemm_bf16_tc_dyt", x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), gemm_splits(M, N, K),
                     sink.resid.data_ptr(), sink.gain.data_ptr(), _ptr(sink.bias), sink.alpha.data_ptr(), normed.data_ptr(), N,
                     _tc(x.device).error.data_ptr(), _stream())
            return Normed(normed, sink.gain)
        sink = None  # the step does not fit: the plain product, and the caller's norm runs as a kernel of its own
    if isinstance(x, RowScaled) or (sink is not None and norm_fusion_ok(x.shape[0], x.dtype, w)
                                    and sink.resid.shape[1] == w.shape[0] and _tma_ok(x, w)):
        return _linear_norm(x, w, out, False, sink)
    _cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype == torch.float32:
        if w.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("linear: a float32 product takes float32 weights and output")
        if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear: operands must be row-major")
        lib.call("ns_gemm_f32", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
                 out.stride(0), _stream())
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported operand types {x.dtype}, {w.dtype}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear: unsupported output type {out.dtype}")
    if USE_TENSOR_CORE_GEMM and (TENSOR_CORE_GEMM_MAX_TOKENS is None or M <= TENSOR_CORE_GEMM_MAX_TOKENS) \
            and linear_tensor_core(x, w, out):
        return out
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return out


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, nq: int,
                  nkv: int, head_dim: int, write_kv: bool = True) -> None:
    """Rotates q and k of the packed [q | k | v] rows in place / into the cache, stores v."""
    _cuda(qkv, positions, token_req, block_table, inv_freq, k_cache, v_cache)
    _i32(positions, "positions"), _i32(token_req, "token_req")
    n = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * head_dim or not qkv.is_contiguous():
        raise KernelError("rope_kv_write: qkv must be contiguous [N, (nq + 2 nkv) * head_dim]")
    if block_table.dtype != torch.int32 or block_table.stride(1) != 1:
        raise KernelError("rope_kv_write: block_table must be int32 with unit inner stride")
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise KernelError("rope_kv_write: inv_freq must be contiguous float32")
    if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("rope_kv_write: cache pages must be contiguous and of the activations' dtype")
    lib.call("ns_rope_kv_write", qkv.data_ptr(), positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), inv_freq.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_size, nq, nkv,
             head_dim, inv_freq.numel(), n, int(bool(write_kv)), dtype_code(qkv.dtype), _stream())


FUSE_ROPE = True  # short steps rotate q and k and write k and v to the cache in the projection's epilogue


def linear_rope(x, w: torch.Tensor, out: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                inv_freq: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, nq: int, nkv: int,
                head_dim: int, write_kv: bool = True) -> bool:
    """The packed [q | k | v] projection with the rotation and the cache write in its epilogue
    (csrc/gemm_tcgen05.cu): out[:, : nq * head_dim] receives the rotated q; k (rotated) and v go to the cache.
    `x` may be a `RowScaled`.  Returns False, having done nothing, when the step or the sizes do not fit
    (more than 64 tokens, a head size other than 32, 64 or 128, features that do not fill tiles of 128, ...)."""
    xt = x.x if isinstance(x, RowScaled) else x
    M, K = xt.shape
    N = w.shape[0]
    if not (FUSE_ROPE and USE_TENSOR_CORE_GEMM and xt.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and 0 < M <= 64
            and (TENSOR_CORE_GEMM_MAX_TOKENS is None or M <= TENSOR_CORE_GEMM_MAX_TOKENS)
            and head_dim in (32, 64, 128) and N == (nq + 2 * nkv) * head_dim and N % 128 == 0 and w.shape[1] == K
            and _tma_ok(xt, w) and out.shape == (M, N) and out.stride(1) == 1 and k_cache.dtype == torch.bfloat16
            and k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.dtype == torch.int32
            and block_table.stride(1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()):
        return False
    _cuda(xt, w, out, positions, token_req, block_table, inv_freq, k_cache, v_cache)
    _i32(positions, "positions"), _i32(token_req, "token_req")
    scaled = x if isinstance(x, RowScaled) else None
    lib.call("ns_gemm_bf16_tc_rope", xt.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, xt.stride(0), w.stride(0),
             out.stride(0), gemm_splits(M, N, K), _ptr(scaled.partials if scaled is not None else None),
             scaled.partials.shape[1] if scaled is not None else 0, scaled.hidden if scaled is not None else 0,
             float(scaled.eps) if scaled is not None else 0.0, positions.data_ptr(), token_req.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), inv_freq.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
             int(page_size), nq, nkv, head_dim, inv_freq.numel(), int(bool(write_kv)), _tc(xt.device).error.data_ptr(), _stream())
    return True


GATE_BLOCK = 64  # gate and up rows alternate in runs of this many in a packed projection that the fused kernel takes


def gated_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, block: int) -> torch.Tensor:
    """out[n, j] = silu(x @ gate_j) * (x @ up_j) for a packed projection w [2I, K]: [gate | up] when
    `block` is 0, runs of `block` gate rows followed by the matching up rows otherwise.  A decode step
    in bfloat16 with block == GATE_BLOCK is one tcgen05 kernel whose epilogue applies the activation;
    everything else is the product into `scratch` [N, 2I] and the swiglu kernel.  `x` may be a `RowScaled`."""
    if isinstance(x, RowScaled):
        if block == GATE_BLOCK and out.dtype == torch.bfloat16:
            return _linear_norm(x, w, out, True, None)
        return swiglu(_linear_norm(x, w, scratch, False, None), out, block)
    _cuda(x, w, out, scratch)
    M, K = x.shape
    if x.dtype == torch.bfloat16 and block == GATE_BLOCK and USE_TENSOR_CORE_GEMM and w.shape[0] % 128 == 0 \
            and TENSOR_CORE_GEMM_MAX_TOKENS is not None and M <= TENSOR_CORE_GEMM_MAX_TOKENS \
            and out.dtype == torch.bfloat16 and not (K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16
                                                     or w.data_ptr() % 16 or x.stride(1) != 1 or w.stride(1) != 1):
        if w.shape[1] != K or out.shape != (M, w.shape[0] // 2) or out.stride(1) != 1:
            raise KernelError(f"gated_linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        lib.call("ns_gemm_bf16_tc_gated", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, w.shape[0], K, x.stride(0),
                 w.stride(0), out.stride(0), 0, gemm_splits(M, w.shape[0], K), _tc(x.device).error.data_ptr(), _stream())
        return out
    return swiglu(linear(x, w, scratch), out, block)


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      token_req: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, nq: int, nkv: int,
                      head_dim: int, page_size: int, scale: float | None = None, window: int = 0,
                      keep_first: int = 0, v_dim: int | None = None, chunk: int = 0, softcap: float = 0.0,
                      sink: torch.Tensor | None = None, gate: torch.Tensor | None = None) -> torch.Tensor:
    """q: [N, >= nq*head_dim] rows (a view into the packed projection is fine, unit inner
    stride); out: [N, nq*v_dim] (`v_dim`: the values' head size when it differs from the keys').  `keep_first`: the
    first so many keys of a request stay visible behind the window.  `chunk` > 0: a query sees only the keys of its own
    chunk of that many positions; `softcap` > 0: scaled scores pass through softcap * tanh(s / softcap).  `sink` and
    `gate`: see `attention`.  See csrc/attention_generic.cu for the masking rule."""
    _cuda(q, k_cache, v_cache, block_table, token_req, positions, out, sink, gate)
    _check_sink_gate(sink, gate, nq, n_rows=out.shape[0], dtype=q.dtype)
    _i32(positions, "positions"), _i32(token_req, "token_req")
    n = out.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[0] != n or q.dtype != out.dtype:
        raise KernelError("attention: q and out must be row-major with the same rows and dtype")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelError("attention: the cache must hold the activations' dtype")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    lib.call("ns_attention_generic_sink", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), token_req.data_ptr(), positions.data_ptr(),
             out.data_ptr(), out.stride(0), n, nq, nkv, head_dim, int(v_dim or head_dim), page_size, float(scale), int(window),
             int(keep_first), int(chunk), float(softcap), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
             dtype_code(q.dtype), _stream())
    return out


def _check_sink_gate(sink: torch.Tensor | None, gate: torch.Tensor | None, nq: int, n_rows: int, dtype: torch.dtype) -> None:
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != nq or not sink.is_contiguous()):
        raise KernelError("attention: the sink is one contiguous float32 number per query head")
    if gate is not None and (gate.dtype != dtype or gate.dim() != 2 or gate.shape[0] != n_rows or gate.shape[1] < nq or gate.stride(1) != 1):
        raise KernelError("attention: the gate is one number per token and query head, in the activations' dtype, unit inner stride")


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                u: torch.Tensor, out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                scratch: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per row of fp32 logits: (token int32, raw log-prob, processed log-prob); `out` gives
    preallocated result tensors (int32, float32, float32, one entry per row) and `scratch` a
    preallocated float32 buffer of 48 floats per row for the kernel's first pass."""
    _cuda(logits, temperature, top_k, top_p, u)
    _i32(top_k, "top_k")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample_rows: logits must be float32 rows")
    for t, name in ((temperature, "temperature"), (top_p, "top_p"), (u, "u")):
        if t.dtype != torch.float32 or t.numel() != rows or not t.is_contiguous():
            raise KernelError(f"sample_rows: {name} must be one contiguous float32 per row")
    if out is not None:
        token, lp_raw, lp_proc = out
        if token.dtype != torch.int32 or lp_raw.dtype != torch.float32 or lp_proc.dtype != torch.float32 \
                or min(token.numel(), lp_raw.numel(), lp_proc.numel()) < rows:
            raise KernelError("sample_rows: out must be (int32, float32, float32) with one entry per row")
    else:
        token = torch.empty(rows, dtype=torch.int32, device=logits.device)
        lp_raw = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lp_proc = torch.empty(rows, dtype=torch.float32, device=logits.device)
    if scratch is None:
        scratch = torch.empty(rows * 48, dtype=torch.float32, device=logits.device)
    elif scratch.dtype != torch.float32 or scratch.numel() < rows * 48 or not scratch.is_contiguous():
        raise KernelError("sample_rows: scratch must be contiguous float32 with 48 entries per row")
    lib.call("ns_sample_rows", logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(),
             top_k.data_ptr(), top_p.data_ptr(), u.data_ptr(), scratch.data_ptr(), token.data_ptr(), lp_raw.data_ptr(),
             lp_proc.data_ptr(), _stream())
    return token, lp_raw, lp_proc


def kv_store(qkv: torch.Tensor, ctx, lane, nq: int, nkv: int, head_dim: int) -> None:
    """Stores k and v of the packed projection at each token's cache slot, unrotated."""
    none = torch.empty(0, dtype=torch.float32, device=qkv.device)
    rope_kv_write(qkv, ctx.positions, ctx.token_req, lane.block_table, none, lane.k, lane.v, lane.page_size, nq, nkv,
                  head_dim, write_kv=True)


TILE_Q = 128         # query rows per block of the m16n8k16 prefill kernel
TILE_Q_TCGEN05 = 256 # and of the tcgen05 one (two tiles of 128)
USE_TCGEN05_ATTENTION = True


def _target_blocks() -> int:
    """Decode attention wants about two blocks per SM before it splits keys further."""
    return 2 * sm_count()


def _tensor_core_attention(dtype: torch.dtype, head_dim: int, v_dim: int | None = None) -> bool:
    """Keys and values of one width: multiples of 16 up to 128; of two widths: multiples of 8, the larger at most 128."""
    if v_dim is None or v_dim == head_dim:
        return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128
    return dtype == torch.bfloat16 and head_dim % 8 == 0 and v_dim % 8 == 0 and 8 <= min(head_dim, v_dim) and max(head_dim, v_dim) <= 128


USE_CLUSTER_DECODE = True


def _cluster_decode_splits(blocks: int, max_kv_len: int | None) -> int:
    """Blocks of one cluster that share a request's keys: a power of two up to 16 that keeps the grid
    within two blocks per SM (measured on a B200: 16 at one request, 4 at 8, 1 at 64, for contexts of
    1,024 and 4,096), and, when the longest context is known, at least two tiles of 64 keys per block."""
    n_splits = 1
    while n_splits < 16 and blocks * n_splits * 2 <= _target_blocks():
        n_splits *= 2
    if max_kv_len is not None:
        while n_splits > 1 and max_kv_len < 128 * n_splits:
            n_splits //= 2
    return n_splits


def attention_decode(qkv: torch.Tensor, lane, ctx, out: torch.Tensor, nq: int, nkv: int, head_dim: int, scale: float,
                     window: int, rows: torch.Tensor | None, n_rows: int, max_kv_len: int | None,
                     work: torch.Tensor | None = None, work_slots: int = 0, keep_first: int = 0, wide_weights: bool = False,
                     chunk: int = 0, softcap: float = 0.0, v_dim: int | None = None, sink: torch.Tensor | None = None,
                     gate: torch.Tensor | None = None) -> None:
    """Split-KV decode attention for the requests that bring one token.  Head sizes 64 and 128 with
    pages of 8 to 64 tokens: TMA loads and a thread-block cluster per request and kv head
    (csrc/attention_decode_tma.cu); everything else: cp.async loads and a merge through global
    memory (csrc/attention_decode.cu).
    `rows`: int32 device tensor of their token rows, or None when every row of the step is one.
    `work` (int32, four per item, from the cache manager's packer) replaces `rows` for the TMA kernel on lanes without
    a window: a request whose context is much longer than the others' comes as several items, a part of its keys
    each, and the kernel adds the parts up through `work_slots` slots of scratch.
    `v_dim`: values of another width than the keys (both multiples of 8): the cp.async kernel, in its instance for the larger."""
    v_dim = head_dim if v_dim is None else v_dim
    head_tiles = -(-(nq // nkv) // 16)
    if window == 0:
        keep_first = 0
    # (kept first keys behind a window, chunks and capped scores are the cp.async kernel's: the TMA kernel loads whole
    # pages in key order and knows one mask)
    if USE_CLUSTER_DECODE and head_dim in (64, 128) and lane.page_size in (8, 16, 32, 64) and qkv.stride(0) % 2 == 0 \
            and not keep_first and not wide_weights and not chunk and not softcap and v_dim == head_dim \
            and sink is None and gate is None:
        n_splits = _cluster_decode_splits(n_rows * nkv * head_tiles, max_kv_len)
        if work is not None and window == 0:
            ws = ctx.workspace
            part = ws.get("attn_work_parts", max(work_slots, 1) * nkv * head_tiles, 16 * head_dim + 32, torch.float32)
            counters = ws.get("attn_work_counters", max(work_slots, 1) * nkv * head_tiles, 1, torch.int32, zero=True)
            lib.call("ns_attention_decode_tma", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
                     lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(),
                     ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), None,
                     work.numel() // 4, nq, nkv, head_dim, lane.page_size, float(scale), 0, n_splits,
                     _tc(qkv.device).error.data_ptr(), work.data_ptr(), part.data_ptr(), counters.data_ptr(), _stream())
            return
        lib.call("ns_attention_decode_tma", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
                 lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(),
                 ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), _ptr(rows), n_rows, nq,
                 nkv, head_dim, lane.page_size, float(scale), int(window), n_splits, _tc(qkv.device).error.data_ptr(),
                 None, None, None, _stream())
        return
    n_splits = max(1, min(16, -(-_target_blocks() // (n_rows * nkv * head_tiles))))
    if max_kv_len is not None:
        # long contexts split further (measured: 4 splits are best at 4,096 keys even for 64 requests),
        # and a split keeps at least two tiles of keys
        n_splits = max(n_splits, min(4, max_kv_len // 1024))
        n_splits = max(1, min(n_splits, -(-max_kv_len // 128)))
        if window > 0:  # ... of the keys that are visible
            n_splits = max(1, min(n_splits, -(-min(max_kv_len, window + keep_first) // 128)))
        if chunk > 0:
            n_splits = max(1, min(n_splits, -(-min(max_kv_len, chunk) // 128)))
    ws = ctx.workspace
    part_o = ws.get("attn_part_o", n_rows * nq * n_splits, -(-max(head_dim, v_dim) // 16) * 16, torch.float32)
    part_ml = ws.get("attn_part_ml", n_rows * nq * n_splits, 2, torch.float32)
    counters = ws.get("attn_counters", n_rows * nkv * head_tiles, 1, torch.int32, zero=True)
    lib.call("ns_attention_decode_kept", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
             lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(), ctx.positions.data_ptr(),
             ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), part_o.data_ptr(), part_ml.data_ptr(),
             counters.data_ptr(), _ptr(rows), n_rows, nq, nkv, head_dim, lane.page_size, float(scale), int(window),
             int(keep_first), int(bool(wide_weights)), int(chunk), float(softcap), n_splits, int(v_dim), _ptr(sink), _ptr(gate),
             gate.stride(0) if gate is not None else 0, _stream())


PREFILL_TWO_HEADS = "auto"  # "always" / "never": tests run both kernels whatever the size of the grid


def attention_prefill(qkv: torch.Tensor, lane, ctx, out: torch.Tensor, nq: int, nkv: int, head_dim: int, scale: float,
                      window: int, tiles: torch.Tensor, tiles_tc: torch.Tensor | None = None, keep_first: int = 0,
                      wide_weights: bool = False, chunk: int = 0, softcap: float = 0.0, v_dim: int | None = None,
                      sink: torch.Tensor | None = None, gate: torch.Tensor | None = None) -> None:
    """Tensor-core attention for portions of prompts.  `tiles`: int32 [n, 2] of (request, offset
    among its tokens of this step).  Head sizes 64 and 128 with pages of 8 to 64 tokens and no window run
    on tcgen05 (csrc/attention_prefill_tc.cu); everything else on m16n8k16 (csrc/attention_prefill.cu), also values of
    another width than the keys (`v_dim`, both multiples of 8)."""
    v_dim = head_dim if v_dim is None else v_dim
    if USE_TCGEN05_ATTENTION and tiles_tc is not None and head_dim in (64, 128) and window == 0 and not wide_weights \
            and not chunk and not softcap and v_dim == head_dim and sink is None and gate is None \
            and lane.page_size in (8, 16, 32, 64) and qkv.stride(0) % 8 == 0 and out.stride(0) % 8 == 0:
        # heads of 64: two query heads of a kv head to a block (four softmax warps per sub-partition keep the exponential
        # unit busier and the keys are read once for both) - once one head to a block would give more blocks than SMs
        two_heads = head_dim == 64 and (nq // nkv) % 2 == 0 and PREFILL_TWO_HEADS != "never" and (
            PREFILL_TWO_HEADS == "always" or nq * tiles_tc.shape[0] > sm_count())
        lib.call("ns_attention_prefill_tc", qkv.data_ptr(), qkv.stride(0), qkv.shape[0], lane.k.data_ptr(),
                 lane.v.data_ptr(), lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0),
                 ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), tiles_tc.data_ptr(), tiles_tc.shape[0], out.data_ptr(),
                 out.stride(0), nq, nkv, head_dim, lane.page_size, float(scale), 2 if two_heads else 1,
                 _tc(qkv.device).error.data_ptr(), _stream())
        return
    lib.call("ns_attention_prefill_kept", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
             lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(),
             tiles.data_ptr(), tiles.shape[0], out.data_ptr(), out.stride(0), nq, nkv, head_dim, lane.page_size,
             float(scale), int(window), int(keep_first) if window else 0, int(bool(wide_weights)), int(chunk), float(softcap), int(v_dim),
             _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, _stream())


def _attention_plan(ctx) -> dict:
    """Once per step: which token rows decode, and the query tiles of the prompt portions."""
    plan = ctx.extras.get("attention_plan")
    if plan is not None:
        return plan
    if ctx.extras.get("graph"):
        plan = {"decode_rows": None, "n_decode": ctx.n_tokens, "tiles": None, "tiles_tc": None, "max_kv_len": None}
    else:
        starts, row = [], 0
        for n in ctx.q_lens:
            starts.append(row)
            row += n
        decode = [s for s, n in zip(starts, ctx.q_lens) if n == 1]
        # the tiles that see the most keys come first: blocks are scheduled in this order
        def make(tile_q):
            ts = [(b, off) for b, n in enumerate(ctx.q_lens) if n > 1 for off in range(0, n, tile_q)]
            ts.sort(key=lambda t: -(ctx.kv_lens[t[0]] - ctx.q_lens[t[0]] + min(t[1] + tile_q, ctx.q_lens[t[0]])))
            return ts
        tiles, tiles_tc = make(TILE_Q), make(TILE_Q_TCGEN05)
        dev = ctx.device
        plan = {
            "n_decode": len(decode),
            "decode_rows": None if len(decode) == ctx.n_tokens or not decode
            else torch.tensor(decode, dtype=torch.int32).to(dev, non_blocking=True),
            "tiles": torch.tensor(tiles, dtype=torch.int32).to(dev, non_blocking=True) if tiles else None,
            "tiles_tc": torch.tensor(tiles_tc, dtype=torch.int32).to(dev, non_blocking=True) if tiles_tc else None,
            "max_kv_len": max((kv for kv, n in zip(ctx.kv_lens, ctx.q_lens) if n == 1), default=None),
        }
    ctx.extras["attention_plan"] = plan
    return plan


def attention(qkv: torch.Tensor, lane, ctx, out: torch.Tensor, nq: int, nkv: int, head_dim: int, scale: float,
              window: int = 0, keep_first: int = 0, v_dim: int | None = None, wide_weights: bool = False, chunk: int = 0,
              softcap: float = 0.0, sink: torch.Tensor | None = None, gate: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of the step's queries (the first nq*head_dim columns of `qkv`) over `lane`.

    bfloat16 with a head size that the tensor-core kernels take: the decode kernel for requests
    that bring one token, the prefill kernel for the others.  `wide_weights`: the softmax weights meet the values
    with about 16 bits each (two bfloat16 products per weight) instead of 8, for designs that state their weights in
    float32; the m16n8k16 kernels have it.  `chunk` > 0: a query sees only the keys of its own chunk of that many
    positions, counted from the start of the sequence; `softcap` > 0: a scaled score s becomes softcap * tanh(s / softcap) (the exact and
    the m16n8k16 kernels); `v_dim`: values of another width than the keys (the same kernels, widths in multiples of 8).
    `sink` (float32 [nq]): the softmax's denominator also holds exp(sink[h]), a term that has no key and no value and counts once
    (zeros: "one added to the denominator"); `gate` ([N, >= nq] in the activations' dtype, a column range of the packed projection
    is fine): head h's output is multiplied by sigmoid(gate[n, h]).  Both run in the exact and the m16n8k16 kernels.  float32, and head
    sizes those kernels refuse: the exact kernel, one warp per (token, head)."""
    v_dim = head_dim if v_dim is None else v_dim
    keep_first = keep_first if window else 0
    if not _tensor_core_attention(qkv.dtype, head_dim, v_dim) or nq // nkv > 64 or (v_dim != head_dim and (nq * head_dim) % 8):
        return attention_generic(qkv, lane.k, lane.v, lane.block_table, ctx.token_req, ctx.positions, out, nq, nkv,
                                 head_dim, lane.page_size, scale, window, keep_first if window else 0, v_dim, chunk, softcap, sink, gate)
    _cuda(qkv, out, lane.k, lane.v, lane.block_table, sink, gate)
    _check_sink_gate(sink, gate, nq, n_rows=out.shape[0], dtype=qkv.dtype)
    if out.stride(1) != 1 or qkv.stride(1) != 1 or lane.k.dtype != qkv.dtype:
        raise KernelError("attention: row-major bfloat16 operands and a bfloat16 cache are needed")
    plan = _attention_plan(ctx)
    both = bool(plan["n_decode"]) and plan["tiles"] is not None
    if both and OVERLAP_MIXED_ATTENTION and not torch.cuda.is_current_stream_capturing():
        # A step of decode tokens beside portions of prompts: the two kernels read the same cache and write different rows.
        # The decode kernel goes to a side stream, so that its blocks fill the SMs which the prefill kernel's last,
        # ragged round of blocks leaves idle instead of running before it on an otherwise empty GPU.
        main = torch.cuda.current_stream()
        side = _side_stream(qkv.device)
        fork, join = _side_events(qkv.device)
        fork.record(main)
        side.wait_event(fork)
        attention_prefill(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["tiles"], plan.get("tiles_tc"), keep_first, wide_weights, chunk, softcap, v_dim, sink, gate)
        with torch.cuda.stream(side):
            attention_decode(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["decode_rows"], plan["n_decode"],
                             plan["max_kv_len"], plan.get("work"), plan.get("work_slots", 0), keep_first, wide_weights, chunk, softcap, v_dim, sink, gate)
            join.record(side)
        main.wait_event(join)
        return out
    if plan["n_decode"]:
        attention_decode(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["decode_rows"], plan["n_decode"],
                         plan["max_kv_len"], plan.get("work"), plan.get("work_slots", 0), keep_first, wide_weights, chunk, softcap, v_dim, sink, gate)
    if plan["tiles"] is not None:
        attention_prefill(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["tiles"], plan.get("tiles_tc"), keep_first, wide_weights, chunk, softcap, v_dim, sink, gate)
    return out


OVERLAP_MIXED_ATTENTION = True
_side: dict = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    st = _side.get((device, "stream"))
    if st is None:
        st = _side[(device, "stream")] = torch.cuda.Stream(device=device)
    return st


def _side_events(device: torch.device):
    ev = _side.get((device, "events"))
    if ev is None:
        ev = _side[(device, "events")] = (torch.cuda.Event(), torch.cuda.Event())
    return ev



# ---- parts that other architectures add: a centred norm, a general rotation, mixers with a state -------------------

def add_layernorm(resid: torch.Tensor, branch: torch.Tensor | None, gain: torch.Tensor, eps: float, out: torch.Tensor,
                  rows: torch.Tensor | None = None, write_resid: bool = True) -> torch.Tensor:
    """resid (+= branch); out = (resid - mean) * rsqrt(var + eps) * gain, statistics in float32 over two passes.
    `rows` as in `add_rmsnorm`."""
    _cuda(resid, branch, gain, out, rows)
    _i32(rows, "rows")
    hidden, n_rows = resid.shape[1], out.shape[0]
    if resid.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("add_layernorm: the residual stream and the gain are float32")
    if not (resid.is_contiguous() and out.is_contiguous() and gain.is_contiguous()) or out.shape[1] != hidden \
            or gain.numel() != hidden:
        raise KernelError("add_layernorm: operands must be contiguous and agree on the width")
    if branch is not None and (branch.dtype != out.dtype or branch.shape != resid.shape or not branch.is_contiguous()):
        raise KernelError("add_layernorm: the branch must match the residual's shape and the output's dtype")
    if rows is None and n_rows != resid.shape[0]:
        raise KernelError("add_layernorm: out and resid differ in rows")
    if rows is not None:
        if rows.numel() != n_rows:
            raise KernelError("add_layernorm: one row index per output row")
        write_resid = False
    lib.call("ns_add_layernorm", resid.data_ptr(), _ptr(branch), gain.data_ptr(), out.data_ptr(), _ptr(rows), n_rows,
             hidden, float(eps), int(bool(write_resid)), dtype_code(out.dtype), _stream())
    return out


def scale_softcap(logits: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32 rows: x * scale, then cap * tanh(x / cap) when cap > 0."""
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("scale_softcap: float32 rows")
    lib.call("ns_scale_softcap", logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0), float(scale),
             float(cap), _stream())
    return logits


def qk_norm_rope_store(qkv: torch.Tensor, ctx, lane, inv_freq: torch.Tensor | None, magnitude: float, interleaved: bool,
                       nq: int, nkv: int, head_dim: int, v_dim: int, q_gain: torch.Tensor | None = None,
                       k_gain: torch.Tensor | None = None, eps: float = 0.0, write_kv: bool = True,
                       bias: torch.Tensor | None = None) -> None:
    """Rows [q: nq*head_dim | k: nkv*head_dim | v: nkv*v_dim]: an RMS norm of the whole q and of the whole k projection
    (when gains are given), a rotation of the first 2 * len(inv_freq) features of each head (pairs (2i, 2i+1) when
    `interleaved`, (i, i + len) otherwise; cos and sin times `magnitude`), q and k rewritten in place, k and v stored at
    the tokens' cache slots when `write_kv` (csrc/rope_kv.cu).  `bias` (float32, one entry per feature of the row): the
    projections' bias, added before the norm.  `nkv` 0: rows of q alone (a mixer that reads another's keys and values)."""
    _cuda(qkv, inv_freq, q_gain, k_gain, bias)
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() != nq * head_dim + nkv * (head_dim + v_dim)):
        raise KernelError("qk_norm_rope_store: a contiguous float32 bias with one entry per feature of [q | k | v]")
    n = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] < nq * head_dim + nkv * (head_dim + v_dim):
        raise KernelError("qk_norm_rope_store: rows of [q | k | v] with unit inner stride")
    for t, name in ((inv_freq, "inv_freq"), (q_gain, "q_gain"), (k_gain, "k_gain")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"qk_norm_rope_store: {name} must be contiguous float32")
    if write_kv:
        if lane.k is None or lane.k.dtype != qkv.dtype or lane.v.dtype != qkv.dtype or not (lane.k.is_contiguous() and lane.v.is_contiguous()):
            raise KernelError("qk_norm_rope_store: cache pages must be contiguous and of the activations' dtype")
        if lane.k.shape[-1] != head_dim or lane.v.shape[-1] != v_dim:
            raise KernelError("qk_norm_rope_store: the cache's head sizes are not the mixer's")
    bt = lane.block_table if write_kv else None
    lib.call("ns_qk_norm_rope_store", qkv.data_ptr(), qkv.stride(0), ctx.positions.data_ptr(), ctx.token_req.data_ptr(),
             _ptr(bt), bt.stride(0) if bt is not None else 0, _ptr(inv_freq), float(magnitude), int(bool(interleaved)),
             inv_freq.numel() if inv_freq is not None else 0, _ptr(q_gain), _ptr(k_gain), float(eps),
             _ptr(lane.k) if write_kv else None, _ptr(lane.v) if write_kv else None, lane.page_size, nq, nkv, head_dim, v_dim, n,
             int(bool(write_kv)), dtype_code(qkv.dtype), _ptr(bias), _stream())


def scan_padded_dim(head_dim: int) -> int:
    """The width that a head of `head_dim` features is padded to in the scan's float32 operands (csrc/recurrent.cu)."""
    for r in (4, 8, 16, 32, 64):
        if 4 * r >= head_dim:
            return 4 * r
    raise KernelError(f"a state mixer's heads hold at most 256 features, not {head_dim}")


def delta_prepare(proj: torch.Tensor, taps: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
                  tail_off: int, ctx, rec: torch.Tensor, kv_heads: int, heads: int, head_dim: int, v_dim: int, off_b: int,
                  off_a: int, q_scale: float, unit_eps: float) -> None:
    """Short convolution + silu over the leading channels of `proj`, unit q and k, decay and write strength, into the
    float32 rows of `rec`; then every request's convolution tail (in `state` at `tail_off`) moves on by this step's tokens."""
    _cuda(proj, taps, a_log, dt_bias, state, rec)
    if rec.dtype != torch.float32 or state.dtype != torch.float32 or taps.dtype != torch.float32 or not taps.is_contiguous() \
            or proj.stride(1) != 1 or rec.stride(1) != 1 or not state.is_contiguous():
        raise KernelError("delta_prepare: float32 taps, state and output; row-major operands")
    lib.call("ns_delta_prepare", proj.data_ptr(), proj.stride(0), taps.data_ptr(), taps.shape[1], a_log.data_ptr(), dt_bias.data_ptr(),
             state.data_ptr(), state.stride(0), int(tail_off), ctx.token_req.data_ptr(), ctx.qo_indptr.data_ptr(),
             ctx.state_slot.data_ptr(), rec.data_ptr(), rec.stride(0), proj.shape[0], ctx.n_requests, kv_heads, heads, head_dim,
             scan_padded_dim(head_dim), v_dim, off_b, off_a, float(q_scale), float(unit_eps), dtype_code(proj.dtype), _stream())


def rotary_prepare(proj: torch.Tensor, ctx, inv_freq: torch.Tensor | None, magnitude: float, interleaved: bool, rec: torch.Tensor,
                   heads: int, head_dim: int, v_dim: int, q_scale: float, k_scale: float) -> None:
    """Rows [q: heads*head_dim | k: heads*head_dim | v: heads*v_dim | ...] of `proj`: q and k rotated by position and scaled, all
    three as float32 into `rec` (heads padded to `scan_padded_dim`)."""
    _cuda(proj, inv_freq, rec)
    if rec.dtype != torch.float32 or proj.stride(1) != 1 or rec.stride(1) != 1:
        raise KernelError("rotary_prepare: float32 output, row-major operands")
    lib.call("ns_rotary_prepare", proj.data_ptr(), proj.stride(0), ctx.positions.data_ptr(), ctx.token_req.data_ptr(), _ptr(inv_freq),
             float(magnitude), int(bool(interleaved)), inv_freq.numel() if inv_freq is not None else 0, rec.data_ptr(), rec.stride(0),
             proj.shape[0], heads, head_dim, scan_padded_dim(head_dim), v_dim, float(q_scale), float(k_scale), dtype_code(proj.dtype),
             _stream())


def linear_scan(rec: torch.Tensor, state: torch.Tensor, ctx, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, v_dim: int,
                decay: torch.Tensor | None = None, gated: bool = False) -> torch.Tensor:
    """The recurrence over each request's tokens of this step (csrc/recurrent.cu).  `rec` rows, as the preparation kernels write
    them: [q: kv_heads*Dp | k: kv_heads*Dp | v: heads*v_dim], then, when `gated` (the delta rule), [g: heads | beta: heads], then
    [k . q: kv_heads]; without `gated`, `decay` [heads] float32.
    `state` [slots, floats] holds S [heads, head_dim, v_dim] at the start of each slot's row; `out` [N, heads*v_dim] float32."""
    _cuda(rec, state, out, decay)
    dp = scan_padded_dim(head_dim)
    off_v = 2 * kv_heads * dp
    off_kq = off_v + heads * v_dim + (2 * heads if gated else 0)
    need = off_kq + kv_heads
    if rec.dtype != torch.float32 or out.dtype != torch.float32 or state.dtype != torch.float32 or rec.shape[1] < need \
            or rec.stride(1) != 1 or out.stride(1) != 1 or not state.is_contiguous() or state.shape[1] < heads * head_dim * v_dim:
        raise KernelError("linear_scan: float32 operands of the sizes the heads need")
    if not gated and (decay is None or decay.dtype != torch.float32 or decay.numel() != heads):
        raise KernelError("linear_scan: one float32 decay per head")
    base = rec.data_ptr()
    g_ptr = base + 4 * (off_v + heads * v_dim) if gated else None
    b_ptr = base + 4 * (off_v + heads * v_dim + heads) if gated else None
    lib.call("ns_linear_scan", base, base + 4 * kv_heads * dp, base + 4 * off_v, g_ptr, b_ptr, base + 4 * off_kq,
             None if gated else decay.data_ptr(),
             rec.stride(0), state.data_ptr(), state.stride(0), ctx.qo_indptr.data_ptr(), ctx.state_slot.data_ptr(), out.data_ptr(),
             out.stride(0), ctx.n_requests, heads, kv_heads, head_dim, v_dim, int(ctx.max_q_len or 1), sm_count(), _stream())
    return out


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor | None, gain: torch.Tensor | None, eps: float, out: torch.Tensor, ctx,
                   heads: int, v_dim: int) -> torch.Tensor:
    """out[n, h, :] = o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps) * gain * silu(gate[n, h, :]); `gate` may be a column range of
    a packed projection, `gain` [v_dim] float32 or None."""
    _cuda(o, gate, gain, out)
    if o.dtype != torch.float32 or o.stride(1) != 1 or out.stride(1) != 1 or (gate is not None and (gate.stride(1) != 1 or gate.dtype != out.dtype)):
        raise KernelError("head_norm_gate: a float32 read-out, row-major operands, the gate in the output's dtype")
    lib.call("ns_head_norm_gate", o.data_ptr(), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(gain), float(eps),
             out.data_ptr(), out.stride(0), ctx.token_req.data_ptr(), o.shape[0], heads, v_dim, dtype_code(out.dtype), _stream())
    return out


# ---- a stream in several copies, a cached latent, routed experts ------------------------------------------------------

def embed_streams(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0, copies: int = 1) -> torch.Tensor:
    """out[n, s * hidden + h] = float(table[ids[n], h]) * scale for each of the `copies` streams."""
    _cuda(table, ids, out)
    _i32(ids, "ids")
    n, hidden = out.shape[0], table.shape[1]
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous() or out.shape[1] != copies * hidden \
            or ids.numel() != n:
        raise KernelError(f"embed_streams: table {tuple(table.shape)}, ids {ids.numel()}, out {tuple(out.shape)}, {copies} copies do not agree")
    lib.call("ns_embed_streams", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, hidden, table.shape[0], float(scale),
             int(copies), dtype_code(table.dtype), _stream())
    return out


def stream_mix_norm(streams: torch.Tensor, n_streams: int, pending: torch.Tensor | None, mix: torch.Tensor | None,
                    out_w: torch.Tensor | None, in_w: torch.Tensor | None, gain: torch.Tensor | None, bias: torch.Tensor | None,
                    eps: float, centered: bool, out: torch.Tensor | None, rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """One pass over each row of `streams` [N, n_streams * H] (float32): the streams take the pending branch
    (x_t = sum_s mix[s, t] x_s + out_w[t] * pending; identity coefficients when None), in place unless `rows` selects
    rows; then out = norm(sum_s in_w[s] x_s) (every stream once when `in_w` is None) with `gain`, optional `bias`,
    RMS or `centered`.  `out` None: only the streams are updated."""
    _cuda(streams, pending, mix, out_w, in_w, gain, bias, out, rows)
    _i32(rows, "rows")
    hidden = streams.shape[1] // n_streams
    if streams.dtype != torch.float32 or not streams.is_contiguous() or streams.shape[1] != n_streams * hidden:
        raise KernelError("stream_mix_norm: the streams are contiguous float32 rows of n_streams * hidden")
    for t, size, name in ((mix, n_streams * n_streams, "mix"), (out_w, n_streams, "out_w"), (in_w, n_streams, "in_w"),
                          (gain, hidden, "gain"), (bias, hidden, "bias")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != size):
            raise KernelError(f"stream_mix_norm: {name} must be contiguous float32 with {size} entries")
    n_rows = streams.shape[0] if rows is None else rows.numel()
    dt = out.dtype if out is not None else pending.dtype if pending is not None else torch.float32
    if out is not None and (out.shape != (n_rows, hidden) or not out.is_contiguous()):
        raise KernelError("stream_mix_norm: out must be contiguous [rows, hidden]")
    if pending is not None and (pending.shape != (streams.shape[0], hidden) or not pending.is_contiguous() or pending.dtype != dt):
        raise KernelError("stream_mix_norm: the pending branch must be [N, hidden], contiguous, of the output's dtype")
    lib.call("ns_stream_mix_norm", streams.data_ptr(), _ptr(pending), _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(gain), _ptr(bias),
             _ptr(out), _ptr(rows), n_rows, int(n_streams), hidden, float(eps), int(bool(centered)), dtype_code(dt), _stream())
    return out


def stream_read(streams: torch.Tensor, n_streams: int, pending: torch.Tensor | None, mix: torch.Tensor | None,
                out_w: torch.Tensor | None, in_w: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    """out [N, H] float32 = sum_s in_w[s] x_s after the pending write, which is applied on the fly and not stored."""
    _cuda(streams, pending, mix, out_w, in_w, out)
    hidden = streams.shape[1] // n_streams
    if out.dtype != torch.float32 or out.shape != (streams.shape[0], hidden) or not out.is_contiguous() or not streams.is_contiguous():
        raise KernelError("stream_read: out must be contiguous float32 [N, hidden]")
    lib.call("ns_stream_read", streams.data_ptr(), _ptr(pending), _ptr(mix), _ptr(out_w), _ptr(in_w), out.data_ptr(),
             streams.shape[0], int(n_streams), hidden, dtype_code(pending.dtype if pending is not None else torch.float32), _stream())
    return out


def latent_rope_store(proj: torch.Tensor, ctx, lane, inv_freq: torch.Tensor | None, magnitude: float, gain: torch.Tensor,
                      eps: float, heads: int, dim: int, rot_dim: int, rank: int, write: bool = True) -> None:
    """Rows [q: heads * (dim + rot_dim) | raw latent: rank | key part: rot_dim | ...]: the rotated parts turn by position
    (pairs (2i, 2i + 1), the first 2 * len(inv_freq) features of a part), q in place; the latent is RMS-normed with
    `gain` and [latent | key part] goes to the token's slot of the lane's cache (csrc/latent.cu)."""
    _cuda(proj, inv_freq, gain, lane.k)
    if proj.stride(1) != 1 or proj.shape[1] < heads * (dim + rot_dim) + rank + rot_dim:
        raise KernelError("latent_rope_store: rows of [q | latent | key part] with unit inner stride")
    if gain.dtype != torch.float32 or gain.numel() != rank or (inv_freq is not None and (inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous())):
        raise KernelError("latent_rope_store: float32 gain of the latent's size and float32 frequencies")
    if write and (lane.k is None or lane.k.dtype != proj.dtype or not lane.k.is_contiguous() or lane.k.shape[-1] != rank + rot_dim
                  or lane.k.shape[-3] != 1):
        raise KernelError("latent_rope_store: the lane's cache must hold one vector of rank + rot_dim features per token")
    bt = lane.block_table
    lib.call("ns_latent_rope_store", proj.data_ptr(), proj.stride(0), ctx.positions.data_ptr(), ctx.token_req.data_ptr(),
             _ptr(bt) if write else None, bt.stride(0) if write else 0, _ptr(inv_freq), float(magnitude),
             inv_freq.numel() if inv_freq is not None else 0, gain.data_ptr(), float(eps), _ptr(lane.k) if write else None,
             lane.page_size, heads, dim, rot_dim, rank, proj.shape[0], int(bool(write)), dtype_code(proj.dtype), _stream())


USE_TENSOR_CORE_LATENT = True
LATENT_BLOCKS_PER_SM = 2  # the tensor-core latent kernel splits a token's keys until the grid holds about this many blocks per SM


def attention_latent(q_lat: torch.Tensor, q_rot: torch.Tensor, lane, ctx, out: torch.Tensor, scale: float, window: int,
                     sink: torch.Tensor | None = None, gate: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of folded queries over a lane of cached latents.  q_lat [N, H, R] and q_rot [N, H, r] (any strides
    with a unit inner one), out [N, H, R] likewise; `sink` [H] float32 joins each head's softmax denominator; `gate`
    [N, H] (raw, a column range of a projection is fine): the head's output times its sigmoid.
    bfloat16 with a latent and a rotated part in multiples of 16 (the latent up to 512): the tensor-core kernel
    (csrc/latent_tc.cu), the keys of a token split over blocks when the step has few tokens; float32 and other sizes:
    the exact kernel (csrc/latent.cu)."""
    _cuda(q_lat, q_rot, out, sink, gate, lane.k)
    n, H, R = q_lat.shape
    r = q_rot.shape[2]
    if q_rot.shape[:2] != (n, H) or out.shape != (n, H, R) or q_lat.stride(2) != 1 or (r and q_rot.stride(2) != 1) or out.stride(2) != 1:
        raise KernelError("attention_latent: q_lat [N, H, R], q_rot [N, H, r], out [N, H, R] with unit inner strides")
    if lane.k.dtype != q_lat.dtype or q_rot.dtype != q_lat.dtype or out.dtype != q_lat.dtype or lane.k.shape[-1] != R + r:
        raise KernelError("attention_latent: operands and cache of one dtype, the cache R + r wide")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != H or not sink.is_contiguous()):
        raise KernelError("attention_latent: one float32 sink per head")
    if gate is not None and (gate.shape != (n, H) or gate.stride(1) != 1 or gate.dtype != q_lat.dtype):
        raise KernelError("attention_latent: gate [N, H] with unit inner stride")
    bt = lane.block_table
    if USE_TENSOR_CORE_LATENT and q_lat.dtype == torch.bfloat16 and R % 16 == 0 and r % 16 == 0 and R <= 512 \
            and out.stride(0) % 2 == 0 and out.stride(1) % 2 == 0 and out.data_ptr() % 4 == 0:
        groups = -(-H // 16)
        blocks = n * groups
        # few (token, head group) pairs: the keys of a token are split over blocks, whole tiles of 64 each
        longest = ctx.max_kv_len or 1
        tiles = -(-(min(window, longest) if window else longest) // 64)
        n_splits = max(1, min(16, tiles, (LATENT_BLOCKS_PER_SM * sm_count()) // blocks))
        part_o = part_ml = None
        if n_splits > 1:
            ws = ctx.workspace
            part_o = ws.get("latent_part_o", blocks * n_splits * 16, R, torch.float32)
            part_ml = ws.get("latent_part_ml", blocks * n_splits * 16, 2, torch.float32)
        lib.call("ns_attention_latent_tc", q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(), q_rot.stride(0),
                 q_rot.stride(1), lane.k.data_ptr(), bt.data_ptr(), bt.stride(0), ctx.token_req.data_ptr(), ctx.positions.data_ptr(),
                 _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0), out.stride(1),
                 _ptr(part_o), _ptr(part_ml), n, H, R, r, lane.page_size, float(scale), int(window), n_splits, _stream())
        return out
    lib.call("ns_attention_latent", q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(), q_rot.stride(0),
             q_rot.stride(1), lane.k.data_ptr(), bt.data_ptr(), bt.stride(0), ctx.token_req.data_ptr(), ctx.positions.data_ptr(),
             _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0), out.stride(1),
             n, H, R, r, lane.page_size, float(scale), int(window), dtype_code(q_lat.dtype), _stream())
    return out


ACTIVATIONS = {"gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu2": 3}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(x) elementwise in float, rounded once: "gelu_erf" (the exact gelu), "gelu_tanh", "silu", "relu2" (the square of relu)."""
    _cuda(x, out)
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: unknown kind {kind!r} (known: {', '.join(ACTIVATIONS)})")
    if x.shape == out.shape and x.dtype == out.dtype and x.dim() == 2 and x.stride(1) == 1 and out.stride(1) == 1 \
            and not (x.is_contiguous() and out.is_contiguous()):
        # column ranges of wider buffers: rows with strides of their own
        lib.call("ns_activation_rows", x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), x.shape[0], x.shape[1], ACTIVATIONS[kind],
                 dtype_code(x.dtype), _stream())
        return out
    if x.shape != out.shape or x.dtype != out.dtype or not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("activation: operands of one shape and dtype, contiguous or rows with unit inner stride")
    lib.call("ns_activation", x.data_ptr(), out.data_ptr(), x.numel(), ACTIVATIONS[kind], dtype_code(x.dtype), _stream())
    return out


def cast_f32(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _cuda(x, out)
    if out.dtype != torch.float32 or out.shape != x.shape or not out.is_contiguous() or x.stride(1) != 1:
        raise KernelError("cast_f32: a contiguous float32 output of the input's shape")
    lib.call("ns_cast_f32", x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], x.shape[1], dtype_code(x.dtype), _stream())
    return out


# the router's logits come from ns_router_logits (every token's block reads the whole router, from L2) while tokens x
# experts x width stays under this; beyond it from the float32 GEMM, which reads the router once per 64 tokens
ROUTER_DIRECT_MAX = 1 << 28


def router_logits(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch=None) -> torch.Tensor:
    """out [N, E] float32 = x @ w^T with float32 products and sums, x in the compute type, w [E, K] float32.  A few tokens:
    one kernel, a warp per (token, expert); many tokens and a large router: x as float32 (into `scratch(...)`'s buffer) and the float32 GEMM."""
    _cuda(x, w, out)
    n, K = x.shape
    E = w.shape[0]
    if w.dtype != torch.float32 or out.dtype != torch.float32 or out.shape != (n, E) or not (w.is_contiguous() and out.is_contiguous()) \
            or x.stride(1) != 1 or w.shape[1] != K:
        raise KernelError("router_logits: float32 router [E, K] and logits [N, E], contiguous; x rows with unit inner stride")
    if n * E * K <= ROUTER_DIRECT_MAX or n <= 64:
        lib.call("ns_router_logits", x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), n, E, K, dtype_code(x.dtype), _stream())
        return out
    x32 = x if x.dtype == torch.float32 else cast_f32(x, scratch(n, K))
    return linear(x32, w, out)


def moe_route(logits: torch.Tensor, groups: int, keep: int, top: int, scale: float, ids: torch.Tensor, weights: torch.Tensor,
              softmax: bool = False) -> None:
    """Per row of float32 logits [N, E]: the chosen experts (int32 [N, top], largest score first) and their weights
    (float32 [N, top]); see csrc/moe.cu for the rule."""
    _cuda(logits, ids, weights)
    n, E = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous() or ids.dtype != torch.int32 or weights.dtype != torch.float32 \
            or ids.shape != (n, top) or weights.shape != (n, top) or not (ids.is_contiguous() and weights.is_contiguous()):
        raise KernelError("moe_route: float32 logits [N, E], int32 ids and float32 weights [N, top], contiguous")
    lib.call("ns_moe_route", logits.data_ptr(), n, E, int(groups), int(keep), int(top), float(scale), int(bool(softmax)),
             ids.data_ptr(), weights.data_ptr(), _stream())


def moe_plan(ids: torch.Tensor, n_experts: int, offsets: torch.Tensor, row_of: torch.Tensor, pair_of: torch.Tensor | None = None) -> None:
    """offsets [E + 1] (running counts per expert), row_of [N, top] (each pair's row where every expert's tokens lie
    side by side) and, when given, pair_of (the pair at each row), all int32."""
    _cuda(ids, offsets, row_of, pair_of)
    for t, name in ((ids, "ids"), (offsets, "offsets"), (row_of, "row_of"), (pair_of, "pair_of")):
        _i32(t, name)
    if offsets.numel() != n_experts + 1 or row_of.numel() != ids.numel() or (pair_of is not None and pair_of.numel() != ids.numel()):
        raise KernelError("moe_plan: offsets [E + 1], row_of and pair_of like ids")
    lib.call("ns_moe_plan", ids.data_ptr(), ids.numel(), int(n_experts), offsets.data_ptr(), row_of.data_ptr(), _ptr(pair_of), _stream())


def moe_grouped_ok(x: torch.Tensor, width: int, ff: int) -> bool:
    """Whether the tensor-core kernel of the grouped experts takes these operands (bfloat16, widths in multiples of 8)."""
    return x.dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0 and x.is_contiguous() and x.data_ptr() % 16 == 0


def moe_grouped(x: torch.Tensor, pair_of: torch.Tensor, offsets: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                w_down: torch.Tensor, act: torch.Tensor, ys: torch.Tensor, top: int) -> torch.Tensor:
    """Every expert over its rows of the plan, on the tensor cores, the counts read on the device (csrc/moe_tc.cu):
    act [pairs, ff] = silu(x . gate) * (x . up), ys [pairs, width] = act . down, both in the plan's row order."""
    _cuda(x, pair_of, offsets, w_gate, w_up, w_down, act, ys)
    n, width = x.shape
    E, ff = w_gate.shape[0], w_gate.shape[1]
    if not all(t.is_contiguous() and t.dtype == torch.bfloat16 for t in (x, w_gate, w_up, w_down, act, ys)) \
            or act.shape != (n * top, ff) or ys.shape != (n * top, width) or w_down.shape != (E, width, ff) or w_up.shape != w_gate.shape:
        raise KernelError("moe_grouped: contiguous bfloat16 operands of the sizes the experts have")
    lib.call("ns_moe_grouped", x.data_ptr(), pair_of.data_ptr(), offsets.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(),
             w_down.data_ptr(), act.data_ptr(), ys.data_ptr(), E, int(top), width, ff, (n * int(top)) // E, _stream())
    return ys


def moe_pad_rows(ids: torch.Tensor, offsets: torch.Tensor, row_of: torch.Tensor, capacity: int) -> None:
    """row_of, in place: from the plan's rows to a layout in which expert e owns rows e * capacity .. (e + 1) * capacity - 1."""
    _cuda(ids, offsets, row_of)
    for t, name in ((ids, "ids"), (offsets, "offsets"), (row_of, "row_of")):
        _i32(t, name)
    lib.call("ns_moe_pad_rows", ids.data_ptr(), offsets.data_ptr(), row_of.data_ptr(), ids.numel(), int(capacity), _stream())


def moe_gather(x: torch.Tensor, row_of: torch.Tensor, xs: torch.Tensor, top: int) -> torch.Tensor:
    """xs[row_of[n, k]] = x[n]; xs may hold more rows than pairs (a padded layout): the others are left as they are."""
    _cuda(x, row_of, xs)
    n, width = x.shape
    if xs.shape[0] < n * top or xs.shape[1] != width or xs.dtype != x.dtype or not (x.is_contiguous() and xs.is_contiguous()):
        raise KernelError("moe_gather: xs [at least N * top, width] of x's dtype, contiguous")
    lib.call("ns_moe_gather", x.data_ptr(), row_of.data_ptr(), xs.data_ptr(), n, int(top), width, dtype_code(x.dtype), _stream())
    return xs


def moe_combine(ys: torch.Tensor, row_of: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, top: int) -> torch.Tensor:
    _cuda(ys, row_of, weights, out)
    n, width = out.shape
    if ys.shape[0] < n * top or ys.shape[1] != width or ys.dtype != out.dtype or not (ys.is_contiguous() and out.is_contiguous()):
        raise KernelError("moe_combine: ys [at least N * top, width] of out's dtype, contiguous")
    lib.call("ns_moe_combine", ys.data_ptr(), row_of.data_ptr(), weights.data_ptr(), out.data_ptr(), n, int(top), width,
             dtype_code(out.dtype), _stream())
    return out


def moe_expert_rows(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                    w_down: torch.Tensor, act: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The chosen experts of a few tokens without a host round trip: w_gate, w_up [E, ff, width], w_down [E, width, ff]."""
    _cuda(x, ids, weights, w_gate, w_up, w_down, act, out)
    n, width = x.shape
    top, ff = ids.shape[1], w_gate.shape[1]
    if not all(t.is_contiguous() for t in (x, ids, weights, w_gate, w_up, w_down, act, out)) or act.shape != (n * top, ff) \
            or out.shape != (n, width) or w_down.shape[1:] != (width, ff) or len({x.dtype, w_gate.dtype, w_up.dtype, w_down.dtype, act.dtype, out.dtype}) != 1:
        raise KernelError("moe_expert_rows: contiguous operands of one dtype and the sizes the experts have")
    lib.call("ns_moe_expert_rows", x.data_ptr(), ids.data_ptr(), weights.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(),
             w_down.data_ptr(), act.data_ptr(), out.data_ptr(), n, top, width, ff, dtype_code(x.dtype), _stream())
    return out


# ---- a norm on a sublayer's output, a token's own gated input, a gate and a bias on rows -------------------------------

def norm_add(resid: torch.Tensor, branch: torch.Tensor | None, gain: torch.Tensor | None, eps: float,
             cast: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> torch.Tensor | None:
    """resid += rmsnorm(branch (+ bias)) * gain, statistics in float32, and `cast` (when given) = the updated rows in its
    own type.  `branch` None: only `cast` is written.  Returns `cast`."""
    _cuda(resid, branch, gain, cast, bias)
    n, hidden = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous():
        raise KernelError("norm_add: the residual stream is contiguous float32")
    dt = branch.dtype if branch is not None else cast.dtype if cast is not None else torch.float32
    if branch is not None and (branch.shape != resid.shape or not branch.is_contiguous() or gain is None
                               or gain.dtype != torch.float32 or gain.numel() != hidden or not gain.is_contiguous()):
        raise KernelError("norm_add: a contiguous branch of the stream's shape and a float32 gain of its width")
    if cast is not None and (cast.shape != resid.shape or not cast.is_contiguous() or cast.dtype != dt):
        raise KernelError("norm_add: the copy must be contiguous, of the stream's shape and the branch's dtype")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != hidden or not bias.is_contiguous()):
        raise KernelError("norm_add: a float32 bias of the stream's width")
    lib.call("ns_norm_add", resid.data_ptr(), _ptr(branch), _ptr(bias), _ptr(gain), _ptr(cast), n, hidden, float(eps), dtype_code(dt),
             _stream())
    return cast


def token_gate(a: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, offset: int, out: torch.Tensor) -> torch.Tensor:
    """out[n, j] = gelu_tanh(a[n, j]) * table[ids[n], offset + j]; a padding row (a negative id) gives zeros."""
    _cuda(a, table, ids, out)
    _i32(ids, "ids")
    n, dim = out.shape
    if a.shape != (n, dim) or a.stride(1) != 1 or table.stride(1) != 1 or not out.is_contiguous() or ids.numel() != n \
            or a.dtype != out.dtype or table.dtype != out.dtype or offset < 0 or offset + dim > table.shape[1]:
        raise KernelError("token_gate: a and out [N, dim] and a table of one dtype whose rows hold offset + dim columns")
    lib.call("ns_token_gate", a.data_ptr(), a.stride(0), table.data_ptr(), table.stride(0), ids.data_ptr(), table.shape[0],
             int(offset), out.data_ptr(), n, dim, dtype_code(out.dtype), _stream())
    return out


def sigmoid_mul(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x *= sigmoid(gate), in place; both [N, C] with unit inner strides (the gate may be a column range of a projection)."""
    _cuda(x, gate)
    if x.shape != gate.shape or x.dim() != 2 or x.stride(1) != 1 or gate.stride(1) != 1 or x.dtype != gate.dtype:
        raise KernelError("sigmoid_mul: rows of one shape and dtype with unit inner strides")
    lib.call("ns_sigmoid_mul", x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), x.shape[0], x.shape[1], dtype_code(x.dtype), _stream())
    return x


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[n, c] += bias[c], in place; `bias` float32."""
    _cuda(x, bias)
    if x.dim() != 2 or x.stride(1) != 1 or bias.dtype != torch.float32 or bias.numel() != x.shape[1] or not bias.is_contiguous():
        raise KernelError("add_bias: rows with a unit inner stride and a float32 bias of their width")
    lib.call("ns_add_bias", x.data_ptr(), x.stride(0), bias.data_ptr(), x.shape[0], x.shape[1], dtype_code(x.dtype), _stream())
    return x


# ---- a norm without statistics; attention whose q and k are prepared head by head -------------------------------------

def add_dyt(resid: torch.Tensor, branches, gain: torch.Tensor, bias: torch.Tensor | None, alpha: torch.Tensor, out: torch.Tensor,
            rows: torch.Tensor | None = None) -> torch.Tensor:
    """resid (+= each of up to two `branches`); out = tanh(alpha * resid) * gain + bias, elementwise in float32 and rounded once
    (csrc/elementwise.cu).  `alpha` is a float32 tensor of one element on the device.  With `rows`, output row j reads input row
    rows[j] and the residual is left unchanged."""
    branches = [b for b in (branches or ()) if b is not None]
    if len(branches) > 2:
        raise KernelError("add_dyt: at most two branches")
    _cuda(resid, gain, bias, alpha, out, rows, *branches)
    _i32(rows, "rows")
    hidden, n_rows = resid.shape[1], out.shape[0]
    if resid.dtype != torch.float32 or gain.dtype != torch.float32 or alpha.dtype != torch.float32 or alpha.numel() != 1 \
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != hidden or not bias.is_contiguous())):
        raise KernelError("add_dyt: the residual stream, the gain, the bias and alpha are float32")
    if not (resid.is_contiguous() and out.is_contiguous() and gain.is_contiguous()) or out.shape[1] != hidden or gain.numel() != hidden:
        raise KernelError("add_dyt: operands must be contiguous and agree on the width")
    for b in branches:
        if b.dtype != out.dtype or b.shape != resid.shape or not b.is_contiguous():
            raise KernelError("add_dyt: a branch must match the residual's shape and the output's dtype")
    if (rows is None and n_rows != resid.shape[0]) or (rows is not None and rows.numel() != n_rows):
        raise KernelError("add_dyt: one output row per residual row, or per selected row")
    a = branches[0] if branches else None
    b = branches[1] if len(branches) > 1 else None
    lib.call("ns_add_dyt", resid.data_ptr(), _ptr(a), _ptr(b), gain.data_ptr(), _ptr(bias), alpha.data_ptr(), out.data_ptr(), _ptr(rows),
             n_rows, hidden, int(rows is None), dtype_code(out.dtype), _stream())
    return out


def head_prepare_store(proj: torch.Tensor, out: torch.Tensor, ctx, lane, nq: int, nkv: int, head_dim: int, v_dim: int, *,
                       inv_freq: torch.Tensor | None = None, magnitude: float = 1.0, interleaved: bool = False,
                       norm: str | None = None, q_gain: torch.Tensor | None = None, k_gain: torch.Tensor | None = None,
                       eps: float = 0.0, q_temp: tuple[float, float] | None = None, taps: torch.Tensor | None = None,
                       v_from_k: bool = False, write_kv: bool = True) -> None:
    """Rows [q: nq*head_dim | k: nkv*head_dim | v: nkv*v_dim] of `proj` (no v part when `v_from_k`: the values are the keys as
    projected), head by head (csrc/head_prepare.cu): a causal convolution over time per channel (`taps` [n, channels] float32, one row
    per tap, the last row the current token's; the last n - 1 inputs of every request live in `lane.state` and move on by this
    step's tokens), an RMS norm per head (`norm`
    "before" or "after" the rotation; gains [head_dim] float32 shared by the heads, or none), the rotation of the first
    2 * len(inv_freq) features (pairs (2i, 2i+1) when `interleaved`, (i, i + len) otherwise; cos and sin times `magnitude`), the
    queries times 1 + coef * ln(floor((position + 1) / every) + 1) for `q_temp` = (coef, every).  q and k go to `out` (which may be
    `proj` itself when there is no convolution), k and v to the tokens' cache slots when `write_kv`."""
    _cuda(proj, out, inv_freq, q_gain, k_gain, taps)
    cols = nq * head_dim + nkv * head_dim + (0 if v_from_k else nkv * v_dim)
    if proj.stride(1) != 1 or out.stride(1) != 1 or proj.shape[1] < cols or out.shape[1] < (nq + nkv) * head_dim \
            or proj.dtype != out.dtype or proj.shape[0] != out.shape[0]:
        raise KernelError("head_prepare_store: rows of [q | k | v] with unit inner stride, in and out of one dtype")
    for t, name, size in ((inv_freq, "inv_freq", None), (q_gain, "q_gain", head_dim), (k_gain, "k_gain", head_dim)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or (size is not None and t.numel() != size)):
            raise KernelError(f"head_prepare_store: {name} must be contiguous float32" + (f" of {size} entries" if size else ""))
    if norm not in (None, "before", "after"):
        raise KernelError(f"head_prepare_store: norm {norm!r} (None, 'before' or 'after' the rotation)")
    n_taps = 1
    state = None
    if taps is not None:
        n_taps = int(taps.shape[0])
        state = lane.state
        if taps.dtype != torch.float32 or not taps.is_contiguous() or taps.dim() != 2 or taps.shape[1] != cols:
            raise KernelError("head_prepare_store: float32 taps, one row per tap over the channels of [q | k | v]")
        if n_taps > 1 and (state is None or state.dtype != torch.float32 or not state.is_contiguous()
                           or state[0].numel() < (n_taps - 1) * cols):
            raise KernelError("head_prepare_store: the convolution's last inputs need a float32 state of (taps - 1) * channels per slot")
        if n_taps > 1 and proj.data_ptr() == out.data_ptr():
            raise KernelError("head_prepare_store: a convolution cannot run in place")
    if write_kv:
        if lane.k is None or lane.v is None or lane.k.dtype != proj.dtype or lane.v.dtype != proj.dtype \
                or not (lane.k.is_contiguous() and lane.v.is_contiguous()):
            raise KernelError("head_prepare_store: cache pages must be contiguous and of the activations' dtype")
        if lane.k.shape[-1] != head_dim or lane.v.shape[-1] != v_dim:
            raise KernelError("head_prepare_store: the cache's head sizes are not the mixer's")
    bt = lane.block_table if write_kv else None
    coef, every = (float(q_temp[0]), float(q_temp[1])) if q_temp else (0.0, 0.0)
    state_floats = state.stride(0) if state is not None and n_taps > 1 else 0
    lib.call("ns_head_prepare_store", proj.data_ptr(), proj.stride(0), out.data_ptr(), out.stride(0), ctx.positions.data_ptr(),
             ctx.token_req.data_ptr(), ctx.qo_indptr.data_ptr(), ctx.state_slot.data_ptr(), _ptr(bt), bt.stride(0) if bt is not None else 0,
             _ptr(inv_freq), float(magnitude), int(bool(interleaved)), inv_freq.numel() if inv_freq is not None else 0, _ptr(q_gain),
             _ptr(k_gain), {None: 0, "before": 1, "after": 2}[norm], float(eps), coef, every, _ptr(taps), n_taps,
             _ptr(state) if n_taps > 1 else None, state_floats, _ptr(lane.k) if write_kv else None, _ptr(lane.v) if write_kv else None,
             lane.page_size, nq, nkv, head_dim, v_dim, int(bool(v_from_k)), proj.shape[0], int(bool(write_kv)), dtype_code(proj.dtype),
             _stream())
    if n_taps > 1:
        lib.call("ns_conv_tail", proj.data_ptr(), proj.stride(0), state.data_ptr(), state_floats, 0, ctx.qo_indptr.data_ptr(),
                 ctx.state_slot.data_ptr(), cols, n_taps, ctx.n_requests, dtype_code(proj.dtype), _stream())
