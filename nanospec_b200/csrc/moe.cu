// Routed experts: scoring and choice per token, the bookkeeping that brings each expert's tokens together, and
// the experts' products for steps of a few tokens.
//
//   ns_cast_f32        rows of the compute type as float (the router's input: its logits are a float product)
//   ns_router_logits   the router's float product for a few tokens (longer steps: ns_cast_f32 and the float GEMM)
//   ns_moe_route       scores = sigmoid(logits) (or softmax); consecutive experts form `groups` groups of equal size, ranked by
//                      the top-2 sum of their scores; all but the `keep` highest-ranked groups are barred; then the `top`
//                      highest-scoring experts that are not barred; weights = score / (sum of the chosen + 1e-20) * scale.
//                      Ties go to the lower index.
//   ns_moe_plan        counts per expert, their running offsets, and for every (token, choice) its row in the
//                      order that has each expert's tokens side by side
//   ns_moe_pad_rows    the same rows in a layout where every expert owns a fixed number of rows (for one batched product)
//   ns_moe_gather      x rows into that order;  ns_moe_combine   out[n] = sum_k weight[n, k] * y[row(n, k)] in float
//   ns_moe_expert_rows the experts themselves for a few tokens, no host round trip: one block row per (token,
//                      choice) streams the chosen expert's gate and up rows, then its down rows
//   ns_activation      out = act(x) elementwise: exact (erf) gelu, tanh gelu, silu, squared relu
#include "common.cuh"

namespace {

template <typename T>
__global__ void cast_f32_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ out, int cols, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / cols;
    out[i] = ns_ld(x, row * ldx + (i - row * cols));
}

constexpr int kMaxExperts = 1024;

// logits[n, e] = x[n] . w[e] in float, for steps of a few tokens: a block per token, its row in shared memory,
// a warp per expert in turn (the sum over the row in a fixed order)
template <typename T>
__global__ void __launch_bounds__(256)
router_logits_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w, float* __restrict__ logits, int E, int K) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float xrow[];
    const int n = blockIdx.x, lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xrow[k] = ns_ld(x, (size_t)n * ldx + k);
    __syncthreads();
    const bool vec = K % 4 == 0 && ((uintptr_t)w % 16 == 0);
    for (int e = wib; e < E; e += 8) {
        const float* wr = w + (size_t)e * K;
        float a = 0.f;
        if (vec) {
            for (int k = lane * 4; k < K; k += 128) {
                const float4 v = *reinterpret_cast<const float4*>(wr + k);
                const float4 u = *reinterpret_cast<const float4*>(xrow + k);
                a = fmaf(v.x, u.x, a); a = fmaf(v.y, u.y, a); a = fmaf(v.z, u.z, a); a = fmaf(v.w, u.w, a);
            }
        } else {
            for (int k = lane; k < K; k += 32) a = fmaf(wr[k], xrow[k], a);
        }
        a = ns_warp_sum(a);
        if (lane == 0) logits[(size_t)n * E + e] = a;
    }
}

// one warp per token
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int n_tokens, int E, int groups, int keep, int top, float scale,
                 int softmax, int* __restrict__ ids, float* __restrict__ weights) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float rs[];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int n = blockIdx.x * 4 + wib;
    if (n >= n_tokens) return;
    float* sc = rs + (size_t)wib * 2 * E;  // scores, then group scores (at most E of them)
    float* gs = sc + E;
    const float* z = logits + (size_t)n * E;
    if (softmax) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = ns_warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(z[e] - mx);
            sc[e] = v;
            sum += v;
        }
        sum = ns_warp_sum(sum);
        for (int e = lane; e < E; e += 32) sc[e] /= sum;
    } else {
        for (int e = lane; e < E; e += 32) sc[e] = 1.f / (1.f + expf(-z[e]));
    }
    __syncwarp();
    const float taken = -1.f;  // scores are positive; a taken or barred entry is marked below every score
    if (groups > 1) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;  // the two largest
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = sc[e];
                if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the best `keep` groups stay; the others' experts are barred
        for (int round = 0; round < groups - keep; ++round) {  // bar the worst, one a round (the higher index at a tie)
            float worst = INFINITY;
            int wi = -1;
            for (int g = lane; g < groups; g += 32) {
                const float v = gs[g];
                if (v >= 0.f && (v < worst || (v == worst && g > wi))) { worst = v; wi = g; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, worst, o);
                const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
                if (oi >= 0 && (wi < 0 || ov < worst || (ov == worst && oi > wi))) { worst = ov; wi = oi; }
            }
            if (lane == 0) gs[wi] = taken;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] < 0.f) sc[e] = taken;
        __syncwarp();
    }
    float total = 0.f, mine = 0.f;
    int mine_id = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = lane; e < E; e += 32) {
            const float v = sc[e];
            if (v > best) { best = v; bi = e; }  // ascending e: the lower index wins a tie
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
        }
        total += best;
        if (lane == k % 32 && k < 32) { mine = best; mine_id = bi; }
        if (k >= 32 && lane == 0) {  // more than 32 choices: written unnormalised, fixed up below
            ids[(size_t)n * top + k] = bi;
            weights[(size_t)n * top + k] = best;
        }
        if (lane == 0) sc[bi] = taken;
        __syncwarp();
    }
    const float f = scale / (total + 1e-20f);
    if (lane < top && lane < 32) {
        ids[(size_t)n * top + lane] = mine_id;
        weights[(size_t)n * top + lane] = mine * f;
    }
    __syncwarp();
    for (int k = 32 + lane; k < top; k += 32) weights[(size_t)n * top + k] *= f;
}

// one block: counts, offsets, rows
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int E, int* __restrict__ offsets, int* __restrict__ row_of,
                int* __restrict__ pair_of) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    __shared__ int count[kMaxExperts], cursor[kMaxExperts];
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = tid; i < n_pairs; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            at += count[e];
        }
        offsets[E] = at;
    }
    __syncthreads();
    // which row of its expert's run a pair gets does not matter to any result: rows are computed alone
    for (int i = tid; i < n_pairs; i += blockDim.x) {
        const int row = atomicAdd(&cursor[ids[i]], 1);
        row_of[i] = row;
        if (pair_of) pair_of[row] = i;
    }
}

// rows of the plan moved to a layout in which every expert owns `capacity` rows: row = expert * capacity + rank in the expert
__global__ void moe_pad_rows_kernel(const int* __restrict__ ids, const int* __restrict__ offsets, int* __restrict__ row_of, int n_pairs,
                                    int capacity) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = ids[i];
    row_of[i] = e * capacity + (row_of[i] - offsets[e]);
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ row_of, T* __restrict__ xs, int top,
                                  int width) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int pair = blockIdx.x;
    const T* src = x + (size_t)(pair / top) * width;
    T* dst = xs + (size_t)row_of[pair] * width;
    for (int h = threadIdx.x; h < width; h += blockDim.x) dst[h] = src[h];
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ ys, const int* __restrict__ row_of, const float* __restrict__ weights,
                                   T* __restrict__ out, int top, int width) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int n = blockIdx.x;
    for (int h = threadIdx.x; h < width; h += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < top; ++k)
            a = fmaf(weights[(size_t)n * top + k], ns_ld(ys, (size_t)row_of[(size_t)n * top + k] * width + h), a);
        ns_st(out, (size_t)n * width + h, a);
    }
}

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ xs, int K, int lane, bool vec) {
    float a = 0.f;
    if (vec) {
        for (int k = lane * 8; k < K; k += 256) {
            float v[8];
            ld8(w + k, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) a = fmaf(v[i], xs[k + i], a);
        }
    } else {
        for (int k = lane; k < K; k += 32) a = fmaf(ns_ld(w, k), xs[k], a);
    }
    return ns_warp_sum(a);
}

// act[pair, j] = silu(gate_e[j] . x) * (up_e[j] . x); grid (pairs, feature chunks), a warp per feature
template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_up_rows_kernel(const T* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ w_gate,
                        const T* __restrict__ w_up, T* __restrict__ act, int top, int width, int ff, int per_block) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float xs[];
    const int pair = blockIdx.x, lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int e = ids[pair];
    const T* xr = x + (size_t)(pair / top) * width;
    for (int k = threadIdx.x; k < width; k += blockDim.x) xs[k] = ns_ld(xr, k);
    __syncthreads();
    const bool vec = width % 8 == 0 && (((uintptr_t)w_gate | (uintptr_t)w_up) % 16 == 0);
    const int j0 = blockIdx.y * per_block, j1 = min(ff, j0 + per_block);
    for (int j = j0 + wib; j < j1; j += 8) {
        const size_t off = ((size_t)e * ff + j) * width;
        const float g = dot_row(w_gate + off, xs, width, lane, vec);
        const float u = dot_row(w_up + off, xs, width, lane, vec);
        if (lane == 0) ns_st(act, (size_t)pair * ff + j, g / (1.f + expf(-g)) * u);
    }
}

// out[n, i] = sum_k weight[n, k] * (down_e(k)[i] . act[n, k]); grid (tokens, feature chunks)
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_rows_kernel(const T* __restrict__ act, const int* __restrict__ ids, const float* __restrict__ weights,
                     const T* __restrict__ w_down, T* __restrict__ out, int top, int width, int ff, int per_block) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float as[];  // [top][ff]
    const int n = blockIdx.x, lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = ns_ld(act, (size_t)n * top * ff + i);
    __syncthreads();
    const bool vec = ff % 8 == 0 && ((uintptr_t)w_down % 16 == 0);
    const int i0 = blockIdx.y * per_block, i1 = min(width, i0 + per_block);
    for (int i = i0 + wib; i < i1; i += 8) {
        float a = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = ids[(size_t)n * top + k];
            a = fmaf(weights[(size_t)n * top + k], dot_row(w_down + ((size_t)e * width + i) * ff, as + (size_t)k * ff, ff, lane, vec), a);
        }
        if (lane == 0) ns_st(out, (size_t)n * width + i, a);
    }
}

__device__ __forceinline__ float act_value(float z, int kind) {
    if (kind == 0) return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
    if (kind == 1) return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    if (kind == 3) { const float p = fmaxf(z, 0.f); return p * p; }
    return z / (1.f + expf(-z));
}

template <typename T>
__global__ void activation_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int kind, size_t total8) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    float v[8];
    ld8(x + i * 8, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = act_value(v[k], kind);
    st8(out + i * 8, v);
}

// rows of `cols` features with strides of their own (column ranges of wider buffers); VEC = 8 needs both rows on 16 bytes
template <typename T, int VEC>
__global__ void activation_rows_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ out, long long ldo, int cols, int kind,
                                       size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int per_row = cols / VEC;
    const size_t row = i / per_row;
    const int c = (int)(i - row * per_row) * VEC;
    if constexpr (VEC == 8) {
        float v[8];
        ld8(x + row * ldx + c, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = act_value(v[k], kind);
        st8(out + row * ldo + c, v);
    } else {
        ns_st(out, row * ldo + c, act_value(ns_ld(x, row * ldx + c), kind));
    }
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, int kind, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    ns_st(out, i, act_value(ns_ld(x, i), kind));
}

}  // namespace

NS_API int ns_cast_f32(const void* x, long long ldx, float* out, int n_rows, int cols, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * cols;
    if (total == 0) return NS_OK;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == NS_F32) NS_LAUNCH((cast_f32_kernel<float>), blocks, 256, 0, stream, (const float*)x, ldx, out, cols, total);
    else if (dtype == NS_BF16) NS_LAUNCH((cast_f32_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (const __nv_bfloat16*)x, ldx, out, cols, total);
    else NS_FAIL(NS_ERR_ARGUMENT, "ns_cast_f32: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_cast_f32");
    return NS_OK;
}

// x [n, K] (row stride ldx) in the compute type, w [E, K] float, logits [n, E] float
NS_API int ns_router_logits(const void* x, long long ldx, const float* w, float* logits, int n_tokens, int E, int K, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 200 * 1024) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_router_logits: a row of %d floats does not fit shared memory", K);
    if (dtype == NS_F32) {
        if (smem > 48 * 1024) NS_CUDA(cudaFuncSetAttribute(router_logits_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        NS_LAUNCH((router_logits_kernel<float>), n_tokens, 256, smem, stream, (const float*)x, ldx, w, logits, E, K);
    } else if (dtype == NS_BF16) {
        if (smem > 48 * 1024) NS_CUDA(cudaFuncSetAttribute(router_logits_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        NS_LAUNCH((router_logits_kernel<__nv_bfloat16>), n_tokens, 256, smem, stream, (const __nv_bfloat16*)x, ldx, w, logits, E, K);
    } else {
        NS_FAIL(NS_ERR_ARGUMENT, "ns_router_logits: unknown dtype %d", dtype);
    }
    NS_CHECK_LAUNCH("ns_router_logits");
    return NS_OK;
}

NS_API int ns_moe_route(const float* logits, int n_tokens, int E, int groups, int keep, int top, float scale, int softmax,
                        int* ids, float* weights, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (E < 1 || E > kMaxExperts || top < 1 || top > E) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_moe_route: %d experts, %d chosen (at most %d experts)", E, top, kMaxExperts);
    if (groups > 1 && (E % groups || keep < 1 || keep > groups || keep * (E / groups) < top))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_moe_route: %d groups over %d experts, %d kept, %d chosen", groups, E, keep, top);
    const size_t smem = (size_t)4 * 2 * E * sizeof(float);
    NS_LAUNCH(moe_route_kernel, (n_tokens + 3) / 4, 128, smem, stream, logits, n_tokens, E, groups, keep, top, scale, softmax, ids, weights);
    NS_CHECK_LAUNCH("ns_moe_route");
    return NS_OK;
}

// pair_of (optional): the inverse of row_of
NS_API int ns_moe_plan(const int* ids, int n_pairs, int E, int* offsets, int* row_of, int* pair_of, cudaStream_t stream) {
    if (E < 1 || E > kMaxExperts) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_moe_plan: %d experts (at most %d)", E, kMaxExperts);
    NS_LAUNCH(moe_plan_kernel, 1, 1024, 0, stream, ids, n_pairs, E, offsets, row_of, pair_of);
    NS_CHECK_LAUNCH("ns_moe_plan");
    return NS_OK;
}

NS_API int ns_moe_pad_rows(const int* ids, const int* offsets, int* row_of, int n_pairs, int capacity, cudaStream_t stream) {
    if (n_pairs <= 0) return NS_OK;
    NS_LAUNCH(moe_pad_rows_kernel, (n_pairs + 255) / 256, 256, 0, stream, ids, offsets, row_of, n_pairs, capacity);
    NS_CHECK_LAUNCH("ns_moe_pad_rows");
    return NS_OK;
}

NS_API int ns_moe_gather(const void* x, const int* row_of, void* xs, int n_tokens, int top, int width, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (dtype == NS_F32) NS_LAUNCH((moe_gather_kernel<float>), n_tokens * top, 128, 0, stream, (const float*)x, row_of, (float*)xs, top, width);
    else if (dtype == NS_BF16) NS_LAUNCH((moe_gather_kernel<__nv_bfloat16>), n_tokens * top, 128, 0, stream, (const __nv_bfloat16*)x, row_of, (__nv_bfloat16*)xs, top, width);
    else NS_FAIL(NS_ERR_ARGUMENT, "ns_moe_gather: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_moe_gather");
    return NS_OK;
}

NS_API int ns_moe_combine(const void* ys, const int* row_of, const float* weights, void* out, int n_tokens, int top, int width,
                          int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (dtype == NS_F32) NS_LAUNCH((moe_combine_kernel<float>), n_tokens, 256, 0, stream, (const float*)ys, row_of, weights, (float*)out, top, width);
    else if (dtype == NS_BF16) NS_LAUNCH((moe_combine_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, (const __nv_bfloat16*)ys, row_of, weights, (__nv_bfloat16*)out, top, width);
    else NS_FAIL(NS_ERR_ARGUMENT, "ns_moe_combine: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_moe_combine");
    return NS_OK;
}

// x [n, width]; ids, weights [n, top]; w_gate, w_up [E, ff, width]; w_down [E, width, ff]; act [n * top, ff] scratch;
// out [n, width]
NS_API int ns_moe_expert_rows(const void* x, const int* ids, const float* weights, const void* w_gate, const void* w_up,
                              const void* w_down, void* act, void* out, int n_tokens, int top, int width, int ff, int dtype,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    const size_t smem_a = (size_t)width * sizeof(float), smem_b = (size_t)top * ff * sizeof(float);
    if (smem_a > 200 * 1024 || smem_b > 200 * 1024)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_moe_expert_rows: a row of %d or %d x %d floats does not fit shared memory", width, top, ff);
    const int per_a = 64, per_b = 64;
    dim3 grid_a(n_tokens * top, (ff + per_a - 1) / per_a), grid_b(n_tokens, (width + per_b - 1) / per_b);
#define NS_MOE_ROWS(T)                                                                                                        \
    {                                                                                                                         \
        if (smem_a > 48 * 1024) NS_CUDA(cudaFuncSetAttribute(moe_gate_up_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); \
        if (smem_b > 48 * 1024) NS_CUDA(cudaFuncSetAttribute(moe_down_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));    \
        NS_LAUNCH((moe_gate_up_rows_kernel<T>), grid_a, 256, smem_a, stream, (const T*)x, ids, (const T*)w_gate, (const T*)w_up,      \
                  (T*)act, top, width, ff, per_a);                                                                            \
        NS_CHECK_LAUNCH("ns_moe_expert_rows");                                                                                \
        NS_LAUNCH((moe_down_rows_kernel<T>), grid_b, 256, smem_b, stream, (const T*)act, ids, weights, (const T*)w_down, (T*)out,     \
                  top, width, ff, per_b);                                                                                     \
    }
    if (dtype == NS_F32) NS_MOE_ROWS(float)
    else if (dtype == NS_BF16) NS_MOE_ROWS(__nv_bfloat16)
    else NS_FAIL(NS_ERR_ARGUMENT, "ns_moe_expert_rows: unknown dtype %d", dtype);
#undef NS_MOE_ROWS
    NS_CHECK_LAUNCH("ns_moe_expert_rows");
    return NS_OK;
}

// the same over rows that lie in wider buffers: x[r * ldx + c] -> out[r * ldo + c], c < cols
NS_API int ns_activation_rows(const void* x, long long ldx, void* out, long long ldo, int n_rows, int cols, int kind, int dtype,
                              cudaStream_t stream) {
    if (n_rows <= 0 || cols <= 0) return NS_OK;
    if (kind < 0 || kind > 3) NS_FAIL(NS_ERR_ARGUMENT, "ns_activation_rows: unknown kind %d", kind);
    if (dtype != NS_F32 && dtype != NS_BF16) NS_FAIL(NS_ERR_ARGUMENT, "ns_activation_rows: unknown dtype %d", dtype);
    const size_t esz = dtype == NS_F32 ? 4 : 2;
    const bool vec = cols % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) % 16 == 0) && (ldx * esz) % 16 == 0 && (ldo * esz) % 16 == 0;
    const size_t total = (size_t)n_rows * (vec ? cols / 8 : cols);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == NS_F32) {
        if (vec) NS_LAUNCH((activation_rows_kernel<float, 8>), blocks, 256, 0, stream, (const float*)x, ldx, (float*)out, ldo, cols, kind, total);
        else NS_LAUNCH((activation_rows_kernel<float, 1>), blocks, 256, 0, stream, (const float*)x, ldx, (float*)out, ldo, cols, kind, total);
    } else {
        if (vec) NS_LAUNCH((activation_rows_kernel<__nv_bfloat16, 8>), blocks, 256, 0, stream, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, cols, kind, total);
        else NS_LAUNCH((activation_rows_kernel<__nv_bfloat16, 1>), blocks, 256, 0, stream, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, cols, kind, total);
    }
    NS_CHECK_LAUNCH("ns_activation_rows");
    return NS_OK;
}

// kind 0: 0.5 z (1 + erf(z / sqrt 2));  1: 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)));  2: z sigmoid(z);  3: max(z, 0)^2
NS_API int ns_activation(const void* x, void* out, long long total, int kind, int dtype, cudaStream_t stream) {
    if (total <= 0) return NS_OK;
    if (kind < 0 || kind > 3) NS_FAIL(NS_ERR_ARGUMENT, "ns_activation: unknown kind %d", kind);
    if (total % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) % 16 == 0)) {  // eight elements to a thread
        const size_t total8 = (size_t)total / 8;
        const unsigned vblocks = (unsigned)((total8 + 255) / 256);
        if (dtype == NS_F32) NS_LAUNCH((activation_vec_kernel<float>), vblocks, 256, 0, stream, (const float*)x, (float*)out, kind, total8);
        else if (dtype == NS_BF16) NS_LAUNCH((activation_vec_kernel<__nv_bfloat16>), vblocks, 256, 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, kind, total8);
        else NS_FAIL(NS_ERR_ARGUMENT, "ns_activation: unknown dtype %d", dtype);
        NS_CHECK_LAUNCH("ns_activation");
        return NS_OK;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == NS_F32) NS_LAUNCH((activation_kernel<float>), blocks, 256, 0, stream, (const float*)x, (float*)out, kind, (size_t)total);
    else if (dtype == NS_BF16) NS_LAUNCH((activation_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, kind, (size_t)total);
    else NS_FAIL(NS_ERR_ARGUMENT, "ns_activation: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_activation");
    return NS_OK;
}
