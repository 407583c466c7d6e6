// Attention over the paged cache, one warp per (token, query head), any head size up to 256.
//
// This is the exact kernel: every score, the softmax and the weighted sum are fp32 with
// accurate expf, and the keys of one query are always visited in the same order (ascending
// from the first key it may see, 32 at a time), so a query's output does not depend on how
// the batch was cut into steps or on what else runs beside it.  The true 32-bit path uses
// it for every step; the bfloat16 path uses it for sizes that the tensor-core kernels refuse.
//
// A query at position p of request r sees the keys at positions max(0, p - window + 1) .. p
// of the same request (window == 0: all of 0 .. p) and, with keep_first > 0, also the keys at
// positions 0 .. keep_first - 1 however far back they lie (they keep their own positions).  With chunk > 0 the
// sequence is cut into chunks of that many positions counted from the start of the sequence and a query sees only the keys of its
// own chunk: the first visible key is then no earlier than floor(p / chunk) * chunk.  With softcap > 0 a score s
// (after the scale) becomes softcap * tanh(s / softcap) before the softmax.  Keys and
// values are read from cache[page, kv_head, offset, :] with page = block_table[r, position / page_size];
// the step's own keys have been written before this kernel runs.  kv_head = q_head / (nq / nkv).
// Keys have d features and values dv (the two caches are separate tensors).
#include "common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;

template <typename T, int DPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ token_req, const int* __restrict__ positions, T* __restrict__ out,
                         int o_stride, int n_tokens, int nq, int nkv, int d, int dv, int page_size, float scale, int window,
                         int keep_first, int chunk, float softcap, const float* __restrict__ sink,
                         const T* __restrict__ gate, int gate_stride) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    extern __shared__ float qsm[];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long w = (long long)blockIdx.x * kWarpsPerBlock + wib;
    if (w >= (long long)n_tokens * nq) return;
    const int n = (int)(w / nq), h = (int)(w % nq);
    T* o = out + (size_t)n * o_stride + (size_t)h * dv;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    const int hk = h / (nq / nkv);
    const int kend = pos + 1;
    int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) kstart = max(kstart, (pos / chunk) * chunk);

    float* qs = qsm + wib * d;
    const T* qrow = q + (size_t)n * q_stride + (size_t)h * d;
    for (int e = lane; e < d; e += 32) qs[e] = ns_ld(qrow, e);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    const int* bt = block_table + (size_t)req * table_stride;

    // two runs of keys: the kept first ones that lie before the window, then the window
    const int kept_end = min(keep_first, kstart);
    for (int seg = 0; seg < 2; ++seg) {
    const int s_lo = seg ? kstart : 0, s_hi = seg ? kend : kept_end;
    for (int kb = s_lo; kb < s_hi; kb += 32) {
        const int key = kb + lane;
        const bool valid = key < s_hi;
        unsigned slot = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[key / page_size];
            // row of cache[page, kv head, offset, :]
            slot = ((unsigned)page * (unsigned)nkv + (unsigned)hk) * (unsigned)page_size + (unsigned)(key % page_size);
            const T* kr = k_cache + (size_t)slot * d;
            float dot = 0.f;
            for (int e = 0; e < d; ++e) dot = fmaf(qs[e], ns_ld(kr, e), dot);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        }
        const float m_new = fmaxf(m, ns_warp_max(s));
        const float corr = expf(m - m_new);  // first chunk: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + ns_warp_sum(p);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        const int cnt = min(32, s_hi - kb);
        for (int j = 0; j < cnt; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const unsigned sj = __shfl_sync(0xffffffffu, slot, j);
            const T* vr = v_cache + (size_t)sj * dv;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < dv) acc[i] = fmaf(pj, ns_ld(vr, e), acc[i]);
            }
        }
        m = m_new;
    }
    }
    if (sink) {  // a term of the denominator that has no key and no value: exp(sink[h])
        const float m_new = fmaxf(m, sink[h]);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sink[h] - m_new);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
    }
    float inv = 1.f / l;
    if (gate) inv *= 1.f / (1.f + expf(-ns_ld(gate, (size_t)n * gate_stride + h)));  // the head's output gate
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int e = lane + 32 * i;
        if (e < dv) ns_st(o, e, acc[i] * inv);
    }
}

template <typename T>
int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
           int table_stride, const int* token_req, const int* positions, void* out, int o_stride, int n_tokens, int nq,
           int nkv, int d, int dv, int page_size, float scale, int window, int keep_first, int chunk, float softcap,
           const float* sink, const void* gate, int gate_stride, cudaStream_t stream) {
    const long long warps = (long long)n_tokens * nq;
    const unsigned blocks = (unsigned)((warps + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const size_t smem = (size_t)kWarpsPerBlock * d * sizeof(float);
    const int dpl = (dv + 31) / 32;
#define NS_ATTN_CASE(D)                                                                                              \
    case D:                                                                                                          \
        NS_LAUNCH((attention_generic_kernel<T, D>), blocks, kWarpsPerBlock * 32, smem, stream,                                \
            (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, table_stride, token_req,       \
            positions, (T*)out, o_stride, n_tokens, nq, nkv, d, dv, page_size, scale, window, keep_first, chunk, softcap, \
            sink, (const T*)gate, gate_stride);                                                                       \
        break;
    switch (dpl) {
        NS_ATTN_CASE(1) NS_ATTN_CASE(2) NS_ATTN_CASE(3) NS_ATTN_CASE(4)
        NS_ATTN_CASE(5) NS_ATTN_CASE(6) NS_ATTN_CASE(7) NS_ATTN_CASE(8)
    }
#undef NS_ATTN_CASE
    NS_CHECK_LAUNCH("ns_attention_generic");
    return NS_OK;
}

}  // namespace

// `sink` (optional, float [nq]): every query's denominator also holds exp(sink[h]), a term without key or value (zeros: "one
// added to the denominator").  `gate` (optional, the activations' type, one number per token and head at
// gate[n * gate_stride + h]): head h's output is multiplied by its sigmoid.
NS_API int ns_attention_generic_sink(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* token_req, const int* positions,
                                void* out, int o_stride, int n_tokens, int nq, int nkv, int d, int dv, int page_size,
                                float scale, int window, int keep_first, int chunk, float softcap, const float* sink,
                                const void* gate, int gate_stride, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (d < 1 || d > 256 || dv < 1 || dv > 256)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_generic: head sizes %d (keys) and %d (values) must lie in 1..256", d, dv);
    if (keep_first < 0 || window < 0 || chunk < 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_generic: window=%d keep_first=%d chunk=%d", window, keep_first, chunk);
    if (chunk > 0 && keep_first > 0) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_generic: kept first keys and chunks do not go together");
    if (nkv < 1 || nq % nkv) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_generic: %d query heads over %d kv heads", nq, nkv);
    if (dtype == NS_F32)
        return launch<float>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions, out,
                             o_stride, n_tokens, nq, nkv, d, dv, page_size, scale, window, keep_first, chunk, softcap, sink, gate, gate_stride, stream);
    if (dtype == NS_BF16)
        return launch<__nv_bfloat16>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions,
                                     out, o_stride, n_tokens, nq, nkv, d, dv, page_size, scale, window, keep_first, chunk, softcap, sink, gate, gate_stride, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_generic: unknown dtype %d", dtype);
}

NS_API int ns_attention_generic(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* token_req, const int* positions,
                                void* out, int o_stride, int n_tokens, int nq, int nkv, int d, int dv, int page_size,
                                float scale, int window, int keep_first, int chunk, float softcap, int dtype, cudaStream_t stream) {
    return ns_attention_generic_sink(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions, out, o_stride,
                                     n_tokens, nq, nkv, d, dv, page_size, scale, window, keep_first, chunk, softcap, nullptr, nullptr,
                                     0, dtype, stream);
}
