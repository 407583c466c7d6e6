// Kernels for layers that norm a sublayer's OUTPUT before it joins the residual stream, and for small gated
// side inputs:
//   ns_norm_add      resid[n] += rmsnorm(branch[n] (+ bias)) * gain, and the updated row once more in the compute
//                    type (the next sublayer reads the stream itself, not a normed copy); without a branch it only
//                    writes that copy
//   ns_token_gate    out[n, j] = gelu_tanh(a[n, j]) * table[ids[n], off + j]: a gate computed from the stream times
//                    a slice of a second embedding row of the token
//   ns_sigmoid_mul   x[n, c] *= sigmoid(g[n, c]) (g may be a column range of a packed projection)
//   ns_add_bias      x[n, c] += bias[c]
// Statistics, sums and the activations are float; results are rounded once.
#include "common.cuh"

namespace {

// One block per row; every thread owns CHUNKS groups of 8 consecutive features (16-byte accesses).
template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS)
norm_add_vec_kernel(float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ bias,
                    const float* __restrict__ gain, T* __restrict__ cast, int hidden, float eps) {
    ns_pdl_launch_dependents();
    __shared__ float scratch[32];
    float g[CHUNKS][8];
    if (branch) {  // the gain is a weight: fetched while the kernel before this one still runs
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int h = (threadIdx.x + c * THREADS) * 8;
            if (h < hidden) ld8(gain + h, g[c]);
        }
    }
    ns_pdl_wait();
    const size_t row = blockIdx.x;
    float* r = resid + row * hidden;
    float v[CHUNKS][8];
    float inv = 0.f;
    if (branch) {
        const T* b = branch + row * hidden;
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int h = (threadIdx.x + c * THREADS) * 8;
            if (h < hidden) {
                ld8(b + h, v[c]);
                if (bias) {
                    float t[8];
                    ld8(bias + h, t);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[c][i] += t[i];
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
            }
        }
        inv = rsqrtf(ns_block_sum(ss, scratch) / (float)hidden + eps);
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int h = (threadIdx.x + c * THREADS) * 8;
        if (h < hidden) {
            float x[8];
            ld8(r + h, x);
            if (branch) {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] += v[c][i] * inv * g[c][i];
                st8(r + h, x);
            }
            if (cast) st8(cast + row * hidden + h, x);
        }
    }
}

// Any width: the branch is read twice (the second time from cache).
template <typename T>
__global__ void __launch_bounds__(256)
norm_add_kernel(float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ bias,
                const float* __restrict__ gain, T* __restrict__ cast, int hidden, float eps) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    __shared__ float scratch[32];
    const size_t row = blockIdx.x;
    float* r = resid + row * hidden;
    const T* b = branch ? branch + row * hidden : nullptr;
    float inv = 0.f;
    if (b) {
        float ss = 0.f;
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
            const float x = ns_ld(b, h) + (bias ? bias[h] : 0.f);
            ss += x * x;
        }
        inv = rsqrtf(ns_block_sum(ss, scratch) / (float)hidden + eps);
    }
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float x = r[h];
        if (b) {
            x += (ns_ld(b, h) + (bias ? bias[h] : 0.f)) * inv * gain[h];
            r[h] = x;
        }
        if (cast) ns_st(cast + row * hidden, h, x);
    }
}

template <typename T>
int launch_norm_add(float* resid, const void* branch, const float* bias, const float* gain, void* cast, int n_rows, int hidden,
                    float eps, cudaStream_t stream) {
    const T* b = (const T*)branch;
    T* c = (T*)cast;
    const bool aligned = hidden % 8 == 0 &&
                         (((uintptr_t)resid | (uintptr_t)branch | (uintptr_t)bias | (uintptr_t)gain | (uintptr_t)cast) % 16 == 0);
    // which kernel runs depends on the width and alignment only, never on the batch
    if (aligned && hidden <= 16384) {
        if (hidden <= 512) NS_LAUNCH((norm_add_vec_kernel<T, 64, 1>), n_rows, 64, 0, stream, resid, b, bias, gain, c, hidden, eps);
        else if (hidden <= 1024) NS_LAUNCH((norm_add_vec_kernel<T, 128, 1>), n_rows, 128, 0, stream, resid, b, bias, gain, c, hidden, eps);
        else if (hidden <= 2048) NS_LAUNCH((norm_add_vec_kernel<T, 128, 2>), n_rows, 128, 0, stream, resid, b, bias, gain, c, hidden, eps);
        else if (hidden <= 4096) NS_LAUNCH((norm_add_vec_kernel<T, 256, 2>), n_rows, 256, 0, stream, resid, b, bias, gain, c, hidden, eps);
        else if (hidden <= 8192) NS_LAUNCH((norm_add_vec_kernel<T, 512, 2>), n_rows, 512, 0, stream, resid, b, bias, gain, c, hidden, eps);
        else NS_LAUNCH((norm_add_vec_kernel<T, 1024, 2>), n_rows, 1024, 0, stream, resid, b, bias, gain, c, hidden, eps);
    } else {
        NS_LAUNCH((norm_add_kernel<T>), n_rows, 256, 0, stream, resid, b, bias, gain, c, hidden, eps);
    }
    NS_CHECK_LAUNCH("ns_norm_add");
    return NS_OK;
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ table, long long ldt,
                                  const int* __restrict__ ids, int vocab, int off, T* __restrict__ out, int dim, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / dim;
    const int j = (int)(i - n * dim);
    const int id = ids[n];
    float e = 0.f;
    if (id >= 0 && id < vocab) e = ns_ld(table, (size_t)id * ldt + off + j);  // a padding row has no token: zero
    ns_st(out, i, gelu_tanh_f(ns_ld(a, n * lda + j)) * e);
}

template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ x, long long ldx, const T* __restrict__ g, long long ldg, int cols, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / cols;
    const int c = (int)(i - n * cols);
    const float z = ns_ld(g, n * ldg + c);
    ns_st(x, n * ldx + c, ns_ld(x, n * ldx + c) * (1.f / (1.f + expf(-z))));
}

// The same two with 8 consecutive features per thread (16-byte accesses in bfloat16): widths, leading sizes and offsets in
// multiples of 8 and pointers on 16 bytes.  Which form runs depends on sizes and alignment only, never on the batch.
template <typename T>
__global__ void token_gate_vec_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ table, long long ldt,
                                      const int* __restrict__ ids, int vocab, int off, T* __restrict__ out, int groups, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / groups;
    const int j = (int)(i - n * groups) * 8;
    const int id = ids[n];
    float e[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, z[8];
    if (id >= 0 && id < vocab) ld8(table + (size_t)id * ldt + off + j, e);
    ld8(a + n * lda + j, z);
#pragma unroll
    for (int k = 0; k < 8; ++k) z[k] = gelu_tanh_f(z[k]) * e[k];
    st8(out + i * 8, z);
}

template <typename T>
__global__ void sigmoid_mul_vec_kernel(T* __restrict__ x, long long ldx, const T* __restrict__ g, long long ldg, int groups, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / groups;
    const int c = (int)(i - n * groups) * 8;
    float z[8], v[8];
    ld8(g + n * ldg + c, z);
    ld8(x + n * ldx + c, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= 1.f / (1.f + expf(-z[k]));
    st8(x + n * ldx + c, v);
}

template <typename T>
int launch_token_gate(const void* a, long long lda, const void* table, long long ldt, const int* ids, int vocab, int off, void* out,
                      int n_rows, int dim, cudaStream_t stream) {
    const bool vec = dim % 8 == 0 && lda % 8 == 0 && ldt % 8 == 0 && off % 8 == 0 &&
                     (((uintptr_t)a | (uintptr_t)table | (uintptr_t)out) % (8 * sizeof(T)) == 0);
    if (vec) {
        const size_t total = (size_t)n_rows * (dim / 8);
        NS_LAUNCH((token_gate_vec_kernel<T>), (unsigned)((total + 127) / 128), 128, 0, stream, (const T*)a, lda, (const T*)table, ldt, ids,
                  vocab, off, (T*)out, dim / 8, total);
    } else {
        const size_t total = (size_t)n_rows * dim;
        NS_LAUNCH((token_gate_kernel<T>), (unsigned)((total + 255) / 256), 256, 0, stream, (const T*)a, lda, (const T*)table, ldt, ids,
                  vocab, off, (T*)out, dim, total);
    }
    NS_CHECK_LAUNCH("ns_token_gate");
    return NS_OK;
}

template <typename T>
int launch_sigmoid_mul(void* x, long long ldx, const void* g, long long ldg, int n_rows, int cols, cudaStream_t stream) {
    const bool vec = cols % 8 == 0 && ldx % 8 == 0 && ldg % 8 == 0 && (((uintptr_t)x | (uintptr_t)g) % (8 * sizeof(T)) == 0);
    if (vec) {
        const size_t total = (size_t)n_rows * (cols / 8);
        NS_LAUNCH((sigmoid_mul_vec_kernel<T>), (unsigned)((total + 127) / 128), 128, 0, stream, (T*)x, ldx, (const T*)g, ldg, cols / 8, total);
    } else {
        const size_t total = (size_t)n_rows * cols;
        NS_LAUNCH((sigmoid_mul_kernel<T>), (unsigned)((total + 255) / 256), 256, 0, stream, (T*)x, ldx, (const T*)g, ldg, cols, total);
    }
    NS_CHECK_LAUNCH("ns_sigmoid_mul");
    return NS_OK;
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, long long ldx, const float* __restrict__ bias, int cols, size_t total) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / cols;
    const int c = (int)(i - n * cols);
    ns_st(x, n * ldx + c, ns_ld(x, n * ldx + c) + bias[c]);
}

}  // namespace

// branch null: only `cast` is written (the stream as it stands, in the compute type).  cast null: only the stream is updated.
NS_API int ns_norm_add(float* resid, const void* branch, const float* bias, const float* gain, void* cast, int n_rows,
                       int hidden, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return NS_OK;
    if (hidden <= 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_norm_add: hidden=%d", hidden);
    if (branch && !gain) NS_FAIL(NS_ERR_ARGUMENT, "ns_norm_add: a branch needs the norm's gain");
    if (!branch && !cast) return NS_OK;
    if (dtype == NS_F32) return launch_norm_add<float>(resid, branch, bias, gain, cast, n_rows, hidden, eps, stream);
    if (dtype == NS_BF16) return launch_norm_add<__nv_bfloat16>(resid, branch, bias, gain, cast, n_rows, hidden, eps, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_norm_add: unknown dtype %d", dtype);
}

NS_API int ns_token_gate(const void* a, long long lda, const void* table, long long ldt, const int* ids, int vocab, int off,
                         void* out, int n_rows, int dim, int dtype, cudaStream_t stream) {
    if ((size_t)n_rows * dim == 0) return NS_OK;
    if (dtype == NS_F32) return launch_token_gate<float>(a, lda, table, ldt, ids, vocab, off, out, n_rows, dim, stream);
    if (dtype == NS_BF16) return launch_token_gate<__nv_bfloat16>(a, lda, table, ldt, ids, vocab, off, out, n_rows, dim, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_token_gate: unknown dtype %d", dtype);
}

NS_API int ns_sigmoid_mul(void* x, long long ldx, const void* g, long long ldg, int n_rows, int cols, int dtype, cudaStream_t stream) {
    if ((size_t)n_rows * cols == 0) return NS_OK;
    if (dtype == NS_F32) return launch_sigmoid_mul<float>(x, ldx, g, ldg, n_rows, cols, stream);
    if (dtype == NS_BF16) return launch_sigmoid_mul<__nv_bfloat16>(x, ldx, g, ldg, n_rows, cols, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_sigmoid_mul: unknown dtype %d", dtype);
}

NS_API int ns_add_bias(void* x, long long ldx, const float* bias, int n_rows, int cols, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * cols;
    if (total == 0) return NS_OK;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == NS_F32)
        NS_LAUNCH((add_bias_kernel<float>), blocks, 256, 0, stream, (float*)x, ldx, bias, cols, total);
    else if (dtype == NS_BF16)
        NS_LAUNCH((add_bias_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (__nv_bfloat16*)x, ldx, bias, cols, total);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_add_bias: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_add_bias");
    return NS_OK;
}
