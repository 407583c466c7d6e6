// Attention over a cached latent: one vector per token, c (R features, RMS-normed) followed by a rotated key
// part (r features) that all heads share.  A head's key is [W_uk c | k_rot] and its value W_uv c; neither is
// ever formed.  The query is folded through W_uk instead (q_lat = W_uk^T q_plain, R features per head), so that
//     score(i, j) = (q_lat_i . c_j + q_rot_i . k_rot_j) * scale
//     o_lat_i     = sum_j p_ij c_j            and the head's output is W_uv o_lat_i,
// which is attention with ONE key head of R + r features whose first R features are also the value.  The two
// folding products are the caller's; this file holds
//   ns_latent_rope_store   per token: RMS norm of the raw latent, rotation of the shared key part and of the
//                          heads' rotated query parts by position, [c | k_rot] written to the token's cache slot
//   ns_attention_latent    the exact kernel: float scores, softmax and sums, keys visited in ascending order from
//                          the first visible one, 32 at a time, whatever the batch looks like.
// Masking: a query at position p sees keys p - window + 1 .. p (window 0: 0 .. p).  A sink (one learned float
// per head) adds exp(sink) to the softmax denominator and nothing to the sum; a gate multiplies a head's
// output by sigmoid(gate) (the projection's raw output is passed).
#include "common.cuh"

namespace {

// ---- preparation ---------------------------------------------------------------------------------
// proj row: [q: H * (d + r) | raw latent: R | key part: r | ...]; the heads' q rows are [d plain | r rotated].
template <typename T>
__global__ void __launch_bounds__(128)
latent_rope_store_kernel(T* __restrict__ proj, int proj_stride, const int* __restrict__ positions,
                         const int* __restrict__ token_req, const int* __restrict__ block_table, int table_stride,
                         const float* __restrict__ inv_freq, float magnitude, int n_pairs, const float* __restrict__ gain,
                         float eps, T* __restrict__ cache, int page_size, int H, int d, int r, int R, int write, int vec) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    __shared__ float scratch[32];
    __shared__ float cs[64], sn[64];  // cos and sin of up to 64 pairs at a time
    const int n = blockIdx.x, tid = threadIdx.x;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    T* row = proj + (size_t)n * proj_stride;
    T* lat = row + (size_t)H * (d + r);
    T* dst = nullptr;
    if (write) {
        const int page = block_table[(size_t)req * table_stride + pos / page_size];
        dst = cache + ((size_t)page * page_size + pos % page_size) * (size_t)(R + r);
    }
    // the latent's norm: two passes, float
    if (write && vec) {  // 8 features per access: every size and offset a multiple of 8, pointers on 16 bytes
        float ss = 0.f;
        for (int e = tid * 8; e < R; e += blockDim.x * 8) {
            float v[8];
            ld8(lat + e, v);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
        }
        const float inv = 1.f / sqrtf(ns_block_sum(ss, scratch) / (float)R + eps);
        for (int e = tid * 8; e < R; e += blockDim.x * 8) {
            float v[8], g[8];
            ld8(lat + e, v);
            ld8(gain + e, g);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = v[k] * inv * g[k];
            st8(dst + e, v);
        }
    } else if (write) {
        float ss = 0.f;
        for (int e = tid; e < R; e += blockDim.x) {
            const float v = ns_ld(lat, e);
            ss += v * v;
        }
        const float inv = 1.f / sqrtf(ns_block_sum(ss, scratch) / (float)R + eps);
        for (int e = tid; e < R; e += blockDim.x) ns_st(dst, e, ns_ld(lat, e) * inv * gain[e]);
    }
    // rotation: pair i of a rotated part is (2i, 2i + 1); features past 2 * n_pairs pass unchanged
    for (int p0 = 0; p0 < n_pairs; p0 += 64) {
        __syncthreads();
        if (tid < 64 && p0 + tid < n_pairs) {
            float s, c;
            sincosf((float)pos * inv_freq[p0 + tid], &s, &c);
            cs[tid] = c * magnitude;
            sn[tid] = s * magnitude;
        }
        __syncthreads();
        const int np = min(64, n_pairs - p0);
        for (int i = tid; i < H * np; i += blockDim.x) {
            const int h = i / np, pi = i % np;
            T* qr = row + (size_t)h * (d + r) + d + 2 * (p0 + pi);
            const float u = ns_ld(qr, 0), v = ns_ld(qr, 1);
            ns_st(qr, 0, u * cs[pi] - v * sn[pi]);
            ns_st(qr, 1, v * cs[pi] + u * sn[pi]);
        }
        if (write)
            for (int pi = tid; pi < np; pi += blockDim.x) {
                const T* kr = lat + R + 2 * (p0 + pi);
                const float u = ns_ld(kr, 0), v = ns_ld(kr, 1);
                ns_st(dst, R + 2 * (p0 + pi), u * cs[pi] - v * sn[pi]);
                ns_st(dst, R + 2 * (p0 + pi) + 1, v * cs[pi] + u * sn[pi]);
            }
    }
    if (write)
        for (int e = 2 * n_pairs + tid; e < r; e += blockDim.x) ns_st(dst, R + e, ns_ld(lat, R + e));
}

// ---- the exact kernel ------------------------------------------------------------------------------
constexpr int kHeadsPerBlock = 8;  // a warp per head; the heads of a block share the staged keys
constexpr int kKeys = 32;

template <typename T, int RPL>
__global__ void __launch_bounds__(kHeadsPerBlock * 32)
attention_latent_kernel(const T* __restrict__ q_lat, long long ql_tok, long long ql_head, const T* __restrict__ q_rot,
                        long long qr_tok, long long qr_head, const T* __restrict__ cache,
                        const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_req,
                        const int* __restrict__ positions, const float* __restrict__ sink, const T* __restrict__ gate,
                        long long gate_tok, T* __restrict__ out, long long o_tok, long long o_head, int H, int R, int r,
                        int page_size, float scale, int window) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float sm[];
    const int D = R + r, DP = D + 1;
    float* tile = sm;                              // [kKeys][DP]
    float* qs = sm + kKeys * DP;                   // [kHeadsPerBlock][D]
    __shared__ unsigned slots[kKeys];
    const int n = blockIdx.x, lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int h = blockIdx.y * kHeadsPerBlock + wib;
    const int req = token_req[n];
    if (req < 0) return;
    const bool live = h < H;
    const int pos = positions[n];
    const int kend = pos + 1;
    const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (live) {
        const T* a = q_lat + (size_t)n * ql_tok + (size_t)h * ql_head;
        const T* b = q_rot + (size_t)n * qr_tok + (size_t)h * qr_head;
        for (int e = lane; e < R; e += 32) qs[wib * D + e] = ns_ld(a, e);
        for (int e = lane; e < r; e += 32) qs[wib * D + R + e] = ns_ld(b, e);
    }
    float m = -INFINITY, l = 0.f;
    float acc[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) acc[i] = 0.f;
    const int* bt = block_table + (size_t)req * table_stride;
    for (int kb = kstart; kb < kend; kb += kKeys) {
        const int cnt = min(kKeys, kend - kb);
        __syncthreads();  // the tile of the round before has been read
        if (threadIdx.x < cnt) {
            const int key = kb + threadIdx.x;
            slots[threadIdx.x] = (unsigned)bt[key / page_size] * (unsigned)page_size + (unsigned)(key % page_size);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < cnt * D; i += blockDim.x) {
            const int j = i / D, e = i - j * D;
            tile[j * DP + e] = ns_ld(cache, (size_t)slots[j] * D + e);
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < cnt) {
            const float* kr = tile + lane * DP;
            const float* qv = qs + wib * D;
            float dot = 0.f;
            for (int e = 0; e < D; ++e) dot = fmaf(qv[e], kr[e], dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, ns_warp_max(s));
        const float corr = expf(m - m_new);
        const float p = lane < cnt ? expf(s - m_new) : 0.f;
        l = l * corr + ns_warp_sum(p);
#pragma unroll
        for (int i = 0; i < RPL; ++i) acc[i] *= corr;
        for (int j = 0; j < cnt; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const float* vr = tile + j * DP;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int e = lane + 32 * i;
                if (e < R) acc[i] = fmaf(pj, vr[e], acc[i]);
            }
        }
        m = m_new;
    }
    if (!live) return;
    float f = 1.f;
    if (sink) {  // the sink joins the denominator only
        const float sk = sink[h];
        const float m_f = fmaxf(m, sk);
        f = expf(m - m_f);
        l = l * f + expf(sk - m_f);
    }
    f /= l;
    if (gate) f *= 1.f / (1.f + expf(-ns_ld(gate, (size_t)n * gate_tok + h)));
    T* o = out + (size_t)n * o_tok + (size_t)h * o_head;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int e = lane + 32 * i;
        if (e < R) ns_st(o, e, acc[i] * f);
    }
}

template <typename T>
int launch_exact(const void* q_lat, long long ql_tok, long long ql_head, const void* q_rot, long long qr_tok,
                 long long qr_head, const void* cache, const int* block_table, int table_stride, const int* token_req,
                 const int* positions, const float* sink, const void* gate, long long gate_tok, void* out, long long o_tok,
                 long long o_head, int n_tokens, int H, int R, int r, int page_size, float scale, int window,
                 cudaStream_t stream) {
    const int D = R + r;
    const size_t smem = ((size_t)kKeys * (D + 1) + (size_t)kHeadsPerBlock * D) * sizeof(float);
    dim3 grid(n_tokens, (H + kHeadsPerBlock - 1) / kHeadsPerBlock);
    const int rpl = (R + 31) / 32;
#define NS_LATENT_CASE(N)                                                                                               \
    {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                           \
            NS_CUDA(cudaFuncSetAttribute(attention_latent_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        NS_LAUNCH((attention_latent_kernel<T, N>), grid, kHeadsPerBlock * 32, smem, stream, (const T*)q_lat, ql_tok, ql_head,   \
                  (const T*)q_rot, qr_tok, qr_head, (const T*)cache, block_table, table_stride, token_req, positions, sink,    \
                  (const T*)gate, gate_tok, (T*)out, o_tok, o_head, H, R, r, page_size, scale, window);                         \
    }
    if (rpl <= 1) NS_LATENT_CASE(1)
    else if (rpl <= 2) NS_LATENT_CASE(2)
    else if (rpl <= 4) NS_LATENT_CASE(4)
    else if (rpl <= 8) NS_LATENT_CASE(8)
    else if (rpl <= 16) NS_LATENT_CASE(16)
    else NS_LATENT_CASE(32)
#undef NS_LATENT_CASE
    NS_CHECK_LAUNCH("ns_attention_latent");
    return NS_OK;
}

}  // namespace

NS_API int ns_latent_rope_store(void* proj, int proj_stride, const int* positions, const int* token_req,
                                const int* block_table, int table_stride, const float* inv_freq, float magnitude,
                                int n_pairs, const float* gain, float eps, void* cache, int page_size, int H, int d, int r,
                                int R, int n_tokens, int write, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (2 * n_pairs > r || n_pairs < 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_latent_rope_store: %d pairs do not fit %d rotated features", n_pairs, r);
    if (write && (!cache || !block_table || !gain)) NS_FAIL(NS_ERR_ARGUMENT, "ns_latent_rope_store: a write needs the cache, the table and the gain");
    // (which form of the norm runs depends on sizes and alignment only, never on the batch)
    const size_t elem = dtype == NS_F32 ? 4 : 2;
    const int vec = R % 8 == 0 && r % 8 == 0 && (H * (d + r)) % 8 == 0 && proj_stride % 8 == 0 &&
                    ((uintptr_t)proj % (8 * elem) == 0) && ((uintptr_t)cache % (8 * elem) == 0) && ((uintptr_t)gain % 16 == 0);
    const int threads = R <= 512 && vec ? 64 : 128;
    if (dtype == NS_F32)
        NS_LAUNCH((latent_rope_store_kernel<float>), n_tokens, threads, 0, stream, (float*)proj, proj_stride, positions, token_req,
                  block_table, table_stride, inv_freq, magnitude, n_pairs, gain, eps, (float*)cache, page_size, H, d, r, R, write, vec);
    else if (dtype == NS_BF16)
        NS_LAUNCH((latent_rope_store_kernel<__nv_bfloat16>), n_tokens, threads, 0, stream, (__nv_bfloat16*)proj, proj_stride, positions,
                  token_req, block_table, table_stride, inv_freq, magnitude, n_pairs, gain, eps, (__nv_bfloat16*)cache, page_size, H,
                  d, r, R, write, vec);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_latent_rope_store: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_latent_rope_store");
    return NS_OK;
}

// q_lat, q_rot, out: element strides per token and per head; gate: one raw value per (token, head), stride per
// token; sink [H] float or null; cache [pages, page_size, R + r].
NS_API int ns_attention_latent(const void* q_lat, long long ql_tok, long long ql_head, const void* q_rot, long long qr_tok,
                               long long qr_head, const void* cache, const int* block_table, int table_stride,
                               const int* token_req, const int* positions, const float* sink, const void* gate,
                               long long gate_tok, void* out, long long o_tok, long long o_head, int n_tokens, int H, int R,
                               int r, int page_size, float scale, int window, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (R < 1 || R > 1024 || r < 0 || R + r > 1280)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_latent: a latent of %d and a rotated part of %d features (at most 1024 and 1280 together)", R, r);
    if (window < 0 || H < 1) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_latent: window=%d heads=%d", window, H);
    if (dtype == NS_F32)
        return launch_exact<float>(q_lat, ql_tok, ql_head, q_rot, qr_tok, qr_head, cache, block_table, table_stride, token_req,
                                   positions, sink, gate, gate_tok, out, o_tok, o_head, n_tokens, H, R, r, page_size, scale, window, stream);
    if (dtype == NS_BF16)
        return launch_exact<__nv_bfloat16>(q_lat, ql_tok, ql_head, q_rot, qr_tok, qr_head, cache, block_table, table_stride,
                                           token_req, positions, sink, gate, gate_tok, out, o_tok, o_head, n_tokens, H, R, r, page_size,
                                           scale, window, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_latent: unknown dtype %d", dtype);
}
