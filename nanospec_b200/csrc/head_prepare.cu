// What lies between an attention mixer's packed projection and its attention kernel when the steps act on one head at
// a time: a short causal convolution over time per channel, an RMS norm per head (before or after the rotation, with a
// gain shared by the heads or without one), the rotation of the leading features of every q and k head, a factor on the
// queries that grows with the position, and the write of keys and values to the token's cache slot.
//
// A row of the projection is [q: nq*d | k: nkv*d | v: nkv*dv]; with `v_from_k` there is no v part and the values are
// the keys as projected (after the convolution, before norm and rotation; dv = d).  In order, per head:
//   1. convolution (`taps` given, [n_taps, C]: one row per tap, so that neighbouring channels' weights lie side by side):
//      y_t[c] = sum_j taps[j, c] * x_(t - n_taps + 1 + j)[c]; inputs before this step's
//      first token of the request come from the request's tail [(n_taps - 1), C] in its state slot, which is zero at a
//      sequence's start.  `ns_conv_tail` (recurrent.cu) moves the tail on afterwards.
//   2. values: stored (v heads, or the k heads' features at this point when v_from_k).
//   3. norm_mode 1: x = x * rsqrt(mean(x^2) + eps) * gain (gain [d] or none), q and k heads.
//   4. rotation of the first 2 * rot_pairs features: interleaved = 1 turns (2i, 2i+1), 0 turns (i, i + rot_pairs);
//      angle = float(position) * inv_freq[i]; cos and sin times `magnitude`.
//   5. norm_mode 2: the norm of step 3, here.
//   6. q heads times 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1)   (temp_every > 0).
//   7. q and k written to `out` (rows laid out like the projection's; it may be the projection itself when there is no
//      convolution), k stored at cache[page, kv head, offset, :].
// One block per token, a warp per head in turn with the head's features in shared memory; everything is float and is
// rounded once, when it is stored.
#include "common.cuh"

namespace {

constexpr int kPrepWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
head_prepare_store_kernel(const T* __restrict__ proj, int ld_proj, T* __restrict__ out, int ld_out,
                          const int* __restrict__ positions, const int* __restrict__ token_req,
                          const int* __restrict__ qo_indptr, const int* __restrict__ state_slot,
                          const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                          float magnitude, int interleaved, int rot_pairs, const float* __restrict__ q_gain,
                          const float* __restrict__ k_gain, int norm_mode, float eps, float temp_coef, float temp_every,
                          const float* __restrict__ taps, int n_taps, const float* __restrict__ state, long long state_floats,
                          T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int nq, int nkv, int d, int dv,
                          int v_from_k, int write_kv, int dmax) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float head_buf[];  // [warp][dmax]
    const int n = blockIdx.x;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* x = head_buf + (size_t)warp * dmax;
    const int C = nq * d + nkv * d + (v_from_k ? 0 : nkv * dv);
    const int start = n_taps > 1 ? qo_indptr[req] : 0;
    const int t = n - start;  // the token's place among the request's tokens of this step
    const float* tail = n_taps > 1 ? state + (long long)state_slot[req] * state_floats : nullptr;
    size_t slot = 0;
    if (write_kv) {
        const int page = block_table[(size_t)req * table_stride + pos / page_size];
        slot = (size_t)page * nkv * page_size + (size_t)(pos % page_size);  // + kv head * page_size
    }
    const float fpos = (float)pos;
    float temp = 1.f;
    if (temp_every > 0.f) temp = 1.f + temp_coef * logf((float)floor((double)(pos + 1) / (double)temp_every) + 1.f);
    const int units = nq + nkv + (v_from_k ? 0 : nkv);
    for (int u = warp; u < units; u += kPrepWarps) {
        const bool is_q = u < nq, is_k = !is_q && u < nq + nkv, is_v = !is_q && !is_k;
        const int hk = is_k ? u - nq : u - nq - nkv;  // the kv head of a k or v unit
        const int col0 = is_v ? (nq + nkv) * d + hk * dv : u * d;
        const int w = is_v ? dv : d;
        __syncwarp();  // the buffer's last use is over
        for (int e = lane; e < w; e += 32) {
            const int c = col0 + e;
            float acc;
            if (taps) {
                acc = 0.f;
                for (int j = 0; j < n_taps; ++j) {
                    const int i = t - (n_taps - 1) + j;
                    const float in = i >= 0 ? ns_ld(proj, (size_t)(start + i) * ld_proj + c) : tail[(size_t)(i + n_taps - 1) * C + c];
                    acc = fmaf(taps[(size_t)j * C + c], in, acc);
                }
            } else {
                acc = ns_ld(proj, (size_t)n * ld_proj + c);
            }
            x[e] = acc;
        }
        __syncwarp();
        if (is_v || (is_k && v_from_k)) {
            if (write_kv) {
                T* vc = v_cache + (slot + (size_t)hk * page_size) * dv;
                for (int e = lane; e < w; e += 32) ns_st(vc, e, x[e]);
            }
            if (is_v) continue;
        }
        const float* gain = is_q ? q_gain : k_gain;
        if (norm_mode == 1) {
            float ss = 0.f;
            for (int e = lane; e < d; e += 32) ss = fmaf(x[e], x[e], ss);
            const float inv = rsqrtf(ns_warp_sum(ss) / (float)d + eps);
            for (int e = lane; e < d; e += 32) x[e] = x[e] * inv * (gain ? gain[e] : 1.f);
            __syncwarp();
        }
        for (int p = lane; p < rot_pairs; p += 32) {
            const int e0 = interleaved ? 2 * p : p, e1 = interleaved ? 2 * p + 1 : p + rot_pairs;
            float sn, cs;
            sincosf(fpos * inv_freq[p], &sn, &cs);
            sn *= magnitude; cs *= magnitude;
            const float a = x[e0], b = x[e1];
            x[e0] = a * cs - b * sn;
            x[e1] = b * cs + a * sn;
        }
        __syncwarp();
        float inv = 1.f;
        if (norm_mode == 2) {
            float ss = 0.f;
            for (int e = lane; e < d; e += 32) ss = fmaf(x[e], x[e], ss);
            inv = rsqrtf(ns_warp_sum(ss) / (float)d + eps);
        }
        T* orow = out + (size_t)n * ld_out + col0;
        T* kc = (is_k && write_kv) ? k_cache + (slot + (size_t)hk * page_size) * d : nullptr;
        for (int e = lane; e < d; e += 32) {
            float y = x[e];
            if (norm_mode == 2) y = y * inv * (gain ? gain[e] : 1.f);
            if (is_q) y *= temp;
            ns_st(orow, e, y);
            if (kc) ns_st(kc, e, y);
        }
    }
}

// The same steps with 16-byte accesses, when heads, rotated parts, rows and caches allow it: a thread holds eight neighbouring
// features of a head in registers, the d / 8 threads of a head are a group of `gs` lanes (a power of two, so that a warp holds whole
// groups), sums over a head are exchanged within the group, and in the halves' pairing a thread gets its partner's features from
// the lane rot_pairs / 8 away.  The token's cosines and sines are computed once, into shared memory, for all of its heads; a block
// per token, every group takes heads in turn.
template <typename T>
__global__ void __launch_bounds__(256)
head_prepare_store_vec_kernel(const T* __restrict__ proj, int ld_proj, T* __restrict__ out, int ld_out,
                              const int* __restrict__ positions, const int* __restrict__ token_req,
                              const int* __restrict__ qo_indptr, const int* __restrict__ state_slot,
                              const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                              float magnitude, int interleaved, int rot_pairs, const float* __restrict__ q_gain,
                              const float* __restrict__ k_gain, int norm_mode, float eps, float temp_coef, float temp_every,
                              const float* __restrict__ taps, int n_taps, const float* __restrict__ state, long long state_floats,
                              T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int nq, int nkv, int d, int dv,
                              int v_from_k, int write_kv, int gs) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int n = blockIdx.x;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    const int C = nq * d + nkv * d + (v_from_k ? 0 : nkv * dv);
    const int start = n_taps > 1 ? qo_indptr[req] : 0;
    const int t = n - start;
    const float* tail = n_taps > 1 ? state + (long long)state_slot[req] * state_floats : nullptr;
    size_t slot = 0;
    if (write_kv) {
        const int page = block_table[(size_t)req * table_stride + pos / page_size];
        slot = (size_t)page * nkv * page_size + (size_t)(pos % page_size);
    }
    const float fpos = (float)pos;
    float temp = 1.f;
    if (temp_every > 0.f) temp = 1.f + temp_coef * logf((float)floor((double)(pos + 1) / (double)temp_every) + 1.f);
    // the token's cosines and sines, once for all heads: [pair][cos, sin], already times the magnitude
    extern __shared__ float cs_sn[];
    for (int p = threadIdx.x; p < rot_pairs; p += blockDim.x) {
        float sn, cs;
        sincosf(fpos * inv_freq[p], &sn, &cs);
        cs_sn[2 * p] = cs * magnitude;
        cs_sn[2 * p + 1] = sn * magnitude;
    }
    __syncthreads();
    const int units = nq + nkv + (v_from_k ? 0 : nkv);
    const int total = units * gs;
    const int lane = threadIdx.x & 31;
    const int rp8 = rot_pairs / 8;  // halves' pairing: the partner chunk lies so many lanes away
    for (int w0 = threadIdx.x - lane; w0 < total; w0 += blockDim.x) {  // the same trips for every lane of a warp
        const int w = w0 + lane;
        const int u = w / gs, c = w - u * gs;  // head unit and chunk of eight features
        const bool is_q = u < nq, is_k = !is_q && u < nq + nkv, is_v = !is_q && !is_k;
        const int hk = is_k ? u - nq : u - nq - nkv;
        const int width = is_v ? dv : d;
        const bool on = u < units && c * 8 < width;
        const int col = (is_v ? (nq + nkv) * d + hk * dv : u * d) + c * 8;
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = 0.f;
        if (on) {
            if (taps) {
                for (int j = 0; j < n_taps; ++j) {
                    const int i2 = t - (n_taps - 1) + j;
                    float in[8], tw[8];
                    if (i2 >= 0) ld8(proj + (size_t)(start + i2) * ld_proj + col, in);
                    else ld8(tail + (size_t)(i2 + n_taps - 1) * C + col, in);
                    ld8(taps + (size_t)j * C + col, tw);
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = fmaf(tw[i], in[i], x[i]);
                }
            } else {
                ld8(proj + (size_t)n * ld_proj + col, x);
            }
            if (write_kv && (is_v || (is_k && v_from_k))) st8(v_cache + (slot + (size_t)hk * page_size) * dv + c * 8, x);
        }
        // (v units go through the exchanges below like the others and store nothing more)
        const float* gain = is_q ? q_gain : k_gain;
        const bool qk = on && !is_v;
        if (norm_mode == 1) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
            for (int o = gs >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = rsqrtf(ss / (float)d + eps);
            if (qk) {
                float g[8];
                if (gain) ld8(gain + c * 8, g);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = x[i] * inv * (gain ? g[i] : 1.f);
            }
        }
        if (rot_pairs > 0) {
            if (interleaved) {
                if (qk && c * 8 < 2 * rot_pairs) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float cs = cs_sn[2 * (c * 4 + i)], sn = cs_sn[2 * (c * 4 + i) + 1];
                        const float a = x[2 * i], b = x[2 * i + 1];
                        x[2 * i] = a * cs - b * sn;
                        x[2 * i + 1] = b * cs + a * sn;
                    }
                }
            } else {
                const bool low = c < rp8, high = !low && c < 2 * rp8;
                const int from = low ? lane + rp8 : lane - rp8;  // the partner's lane (unused outside the rotated part)
                float y[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = __shfl_sync(0xffffffffu, x[i], (low || high) ? from : lane);
                if (qk && (low || high)) {
                    const int p0 = (low ? c : c - rp8) * 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float cs = cs_sn[2 * (p0 + i)], sn = cs_sn[2 * (p0 + i) + 1];
                        x[i] = low ? x[i] * cs - y[i] * sn : x[i] * cs + y[i] * sn;
                    }
                }
            }
        }
        if (norm_mode == 2) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
            for (int o = gs >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = rsqrtf(ss / (float)d + eps);
            if (qk) {
                float g[8];
                if (gain) ld8(gain + c * 8, g);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = x[i] * inv * (gain ? g[i] : 1.f);
            }
        }
        if (qk) {
            if (is_q) {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] *= temp;
            }
            st8(out + (size_t)n * ld_out + col, x);
            if (is_k && write_kv) st8(k_cache + (slot + (size_t)hk * page_size) * d + c * 8, x);
        }
    }
}

}  // namespace

NS_API int ns_head_prepare_store(const void* proj, int ld_proj, void* out, int ld_out, const int* positions, const int* token_req,
                                 const int* qo_indptr, const int* state_slot, const int* block_table, int table_stride,
                                 const float* inv_freq, float magnitude, int interleaved, int rot_pairs, const float* q_gain,
                                 const float* k_gain, int norm_mode, float eps, float temp_coef, float temp_every,
                                 const float* taps, int n_taps, const float* state, long long state_floats, void* k_cache,
                                 void* v_cache, int page_size, int nq, int nkv, int d, int dv, int v_from_k, int n_tokens,
                                 int write_kv, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (rot_pairs < 0 || 2 * rot_pairs > d) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_head_prepare_store: %d pairs in a head of %d", rot_pairs, d);
    if (rot_pairs > 0 && !inv_freq) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: no frequencies");
    if (norm_mode < 0 || norm_mode > 2) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: norm_mode=%d", norm_mode);
    if (v_from_k && dv != d) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: keys that double as values have one width (%d, %d)", d, dv);
    if (write_kv && (!k_cache || !v_cache || !block_table)) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: no cache to write");
    if (taps && n_taps < 1) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: %d taps", n_taps);
    if (!taps) n_taps = 1;
    if (n_taps > 1 && (!state || !qo_indptr || !state_slot)) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: a convolution over several tokens needs a state");
    if (n_taps > 1 && proj == out) NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: a convolution cannot run in place");
    const int dmax = d > dv ? d : dv;
    // 16-byte accesses: heads, the rotated part (in the halves' pairing also each half), rows and caches in multiples of eight features
    int gs = 1;
    while (gs * 8 < dmax) gs *= 2;
    const bool vec = d % 8 == 0 && dv % 8 == 0 && gs <= 32 && ld_proj % 8 == 0 && ld_out % 8 == 0 && (2 * rot_pairs) % 8 == 0 &&
                     (interleaved || rot_pairs % 8 == 0) &&
                     (((uintptr_t)proj | (uintptr_t)out | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)state | (uintptr_t)taps |
                       (write_kv ? ((uintptr_t)k_cache | (uintptr_t)v_cache) : 0)) % 16 == 0) &&
                     (n_taps <= 1 || state_floats % 4 == 0);
    if (vec) {
        const int units = nq + nkv + (v_from_k ? 0 : nkv);
        const int lanes = units * gs;
        const int threads = lanes >= 256 ? 256 : ((lanes + 31) / 32) * 32;
        const size_t rot_smem = (size_t)2 * rot_pairs * sizeof(float);
        if (dtype == NS_F32)
            NS_LAUNCH((head_prepare_store_vec_kernel<float>), n_tokens, threads, rot_smem, stream, (const float*)proj, ld_proj, (float*)out,
                      ld_out, positions, token_req, qo_indptr, state_slot, block_table, table_stride, inv_freq, magnitude, interleaved,
                      rot_pairs, q_gain, k_gain, norm_mode, eps, temp_coef, temp_every, taps, n_taps, state, state_floats,
                      (float*)k_cache, (float*)v_cache, page_size, nq, nkv, d, dv, v_from_k, write_kv, gs);
        else if (dtype == NS_BF16)
            NS_LAUNCH((head_prepare_store_vec_kernel<__nv_bfloat16>), n_tokens, threads, rot_smem, stream, (const __nv_bfloat16*)proj,
                      ld_proj, (__nv_bfloat16*)out, ld_out, positions, token_req, qo_indptr, state_slot, block_table, table_stride,
                      inv_freq, magnitude, interleaved, rot_pairs, q_gain, k_gain, norm_mode, eps, temp_coef, temp_every, taps, n_taps,
                      state, state_floats, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_size, nq, nkv, d, dv, v_from_k,
                      write_kv, gs);
        else
            NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: unknown dtype %d", dtype);
        NS_CHECK_LAUNCH("ns_head_prepare_store");
        return NS_OK;
    }
    const size_t smem = (size_t)kPrepWarps * dmax * sizeof(float);
    if (smem > 48 * 1024) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_head_prepare_store: heads of %d features", dmax);
    if (dtype == NS_F32)
        NS_LAUNCH((head_prepare_store_kernel<float>), n_tokens, kPrepWarps * 32, smem, stream, (const float*)proj, ld_proj, (float*)out,
                  ld_out, positions, token_req, qo_indptr, state_slot, block_table, table_stride, inv_freq, magnitude, interleaved,
                  rot_pairs, q_gain, k_gain, norm_mode, eps, temp_coef, temp_every, taps, n_taps, state, state_floats,
                  (float*)k_cache, (float*)v_cache, page_size, nq, nkv, d, dv, v_from_k, write_kv, dmax);
    else if (dtype == NS_BF16)
        NS_LAUNCH((head_prepare_store_kernel<__nv_bfloat16>), n_tokens, kPrepWarps * 32, smem, stream, (const __nv_bfloat16*)proj,
                  ld_proj, (__nv_bfloat16*)out, ld_out, positions, token_req, qo_indptr, state_slot, block_table, table_stride,
                  inv_freq, magnitude, interleaved, rot_pairs, q_gain, k_gain, norm_mode, eps, temp_coef, temp_every, taps, n_taps,
                  state, state_floats, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_size, nq, nkv, d, dv, v_from_k,
                  write_kv, dmax);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_head_prepare_store: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_head_prepare_store");
    return NS_OK;
}
