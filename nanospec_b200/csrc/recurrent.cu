// Mixers with a fixed-size state per request: linear attention with a decay (retention) and the gated
// delta rule, for portions of prompts and single decoded tokens alike.
//
// Per head the state is a matrix S [D, V] of floats.  For every token, in order:
//     plain:  S = g S + k v^T                      o = S^T q
//     delta:  S = g S;  u = beta (v - S^T k);  S = S + k u^T;   o = S^T q
// The read-out is taken from the state before the token's write, which is the same number:
//     o = S_new^T q = g (S_old^T q) + w (k . q)      with w = v (plain) or u (delta),
// so that the two sums over a column, S_old^T k and S_old^T q, run side by side and the write to S is off the path
// from one token to the next; k . q per token and key head comes from the preparation.
// The columns of S never meet: column e needs only v[e], so the scan runs one column per group of four
// lanes (each lane holds a quarter of the column's D entries in registers), walks the request's tokens of
// this step in order, and leaves the state where the next step finds it.  A request's result therefore
// does not depend on how its tokens were cut into steps: the operations per token are the same.
//
// Everything that enters the recurrence is prepared in float by a kernel with one block per token
// (`*_prepare`): q, k (a head's row padded with zeros to a multiple of 4 * R floats), v, and for the delta
// rule the decay and the write strength.  A third kernel divides each head's read-out by its root mean
// square, applies a gain and the output gate, and rounds once.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
template <typename T> __device__ __forceinline__ float round_to(float x);
template <> __device__ __forceinline__ float round_to<float>(float x) { return x; }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---------------------------------------------------------------------------------------
// delta rule, preparation.  proj row: the packed projection [q: G*D | k: G*D | v: H*V | ...] with the
// write-strength and decay inputs at columns off_b and off_a (H each).  The C = 2*G*D + H*V leading columns
// pass a causal convolution over time per channel (taps [C, n_taps], the last tap is the current token's;
// inputs before this step's first token come from the request's tail [(n_taps - 1), C] in its state, which
// is zero at a sequence's start) and silu; the result is rounded to the activations' type.  Then q and k
// become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale, and
//     g = exp(-exp(A_log[h]) * softplus(a + dt_bias[h])),  beta = sigmoid(b).
// rec row (floats): [q: G*Dp | k: G*Dp | v: H*V | g: H | beta: H | k . q: G].
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ proj, int ld_proj, const float* __restrict__ taps, int n_taps,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     long long state_floats, long long tail_off, const int* __restrict__ token_req,
                     const int* __restrict__ qo_indptr, const int* __restrict__ state_slot, float* __restrict__ rec, int ld_rec,
                     int G, int H, int D, int Dp, int V, int off_b, int off_a, float q_scale, float unit_eps) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    extern __shared__ float ch[];  // the C channels after convolution and silu
    const int n = blockIdx.x;
    const int req = token_req[n];
    if (req < 0) return;
    const int start = qo_indptr[req], t = n - start;
    const int C = 2 * G * D + H * V;
    const float* tail = state + (long long)state_slot[req] * state_floats + tail_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n_taps; ++j) {
            const int i = t - (n_taps - 1) + j;
            const float x = i >= 0 ? ns_ld(proj, (size_t)(start + i) * ld_proj + c) : tail[(size_t)(i + n_taps - 1) * C + c];
            acc = fmaf(taps[(size_t)c * n_taps + j], x, acc);
        }
        ch[c] = round_to<T>(silu_f(acc));
    }
    __syncthreads();
    float* out = rec + (size_t)n * ld_rec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float* kq = out + (size_t)2 * G * Dp + (size_t)H * V + 2 * H;
    for (int hd = warp; hd < G; hd += nwarp) {  // q head hd and k head hd
        const float* xq = ch + hd * D;
        const float* xk = ch + (G + hd) * D;
        float sq = 0.f, sk = 0.f, qk = 0.f;
        for (int e = lane; e < D; e += 32) { sq += xq[e] * xq[e]; sk += xk[e] * xk[e]; }
        const float inv_q = rsqrtf(ns_warp_sum(sq) + unit_eps) * q_scale, inv_k = rsqrtf(ns_warp_sum(sk) + unit_eps);
        float* oq = out + (size_t)hd * Dp;
        float* ok = out + (size_t)(G + hd) * Dp;
        for (int e = lane; e < Dp; e += 32) {
            const float a = e < D ? xq[e] * inv_q : 0.f, b = e < D ? xk[e] * inv_k : 0.f;
            oq[e] = a; ok[e] = b;
            qk = fmaf(a, b, qk);
        }
        qk = ns_warp_sum(qk);
        if (lane == 0) kq[hd] = qk;
    }
    float* ov = out + (size_t)2 * G * Dp;
    for (int e = threadIdx.x; e < H * V; e += blockDim.x) ov[e] = ch[2 * G * D + e];
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float a = ns_ld(proj, (size_t)n * ld_proj + off_a + h) + dt_bias[h];
        const float b = ns_ld(proj, (size_t)n * ld_proj + off_b + h);
        ov[H * V + h] = expf(-expf(a_log[h]) * softplus_f(a));
        ov[H * V + H + h] = 1.f / (1.f + expf(-b));
    }
}

// After the preparation: the tail of every request moves on by the tokens of this step.
// new tail[j] = the input at (L - (n_taps - 1) + j) of the step's L tokens, or the old tail[j + L] before them.
template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ proj, int ld_proj, float* __restrict__ state, long long state_floats,
                                 long long tail_off, const int* __restrict__ qo_indptr, const int* __restrict__ state_slot,
                                 int C, int n_taps) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int start = qo_indptr[b], L = qo_indptr[b + 1] - start;
    if (L <= 0) return;
    float* tail = state + (long long)state_slot[b] * state_floats + tail_off;
    for (int j = 0; j < n_taps - 1; ++j) {  // ascending: entry j + L is read before it is written
        const int i = L - (n_taps - 1) + j;
        tail[(size_t)j * C + c] = i >= 0 ? ns_ld(proj, (size_t)(start + i) * ld_proj + c) : tail[(size_t)(j + L) * C + c];
    }
}

// ---------------------------------------------------------------------------------------
// linear attention, preparation.  proj row: [q: H*D | k: H*D | v: H*V | ...].  q and k are rotated by the
// token's position on the first 2 * rot_pairs features of each head (interleaved = 1: pairs (2i, 2i+1); 0:
// pairs (i, i + rot_pairs); angle = float(position) * inv_freq[i]; cos and sin times `magnitude`), then k is
// multiplied by k_scale and q by q_scale.  rec row (floats): [q: H*Dp | k: H*Dp | v: H*V | k . q: H].
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rotary_prepare_kernel(const T* __restrict__ proj, int ld_proj, const int* __restrict__ positions, const int* __restrict__ token_req,
                      const float* __restrict__ inv_freq, float magnitude, int interleaved, int rot_pairs, float* __restrict__ rec,
                      int ld_rec, int H, int D, int Dp, int V, float q_scale, float k_scale) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int n = blockIdx.x;
    if (token_req[n] < 0) return;
    const float fpos = (float)positions[n];
    const T* row = proj + (size_t)n * ld_proj;
    float* out = rec + (size_t)n * ld_rec;
    const int units = rot_pairs + (Dp - 2 * rot_pairs);
    for (int w = threadIdx.x; w < 2 * H * units; w += blockDim.x) {
        const int hd = w / units, u = w - hd * units;  // q heads, then k heads
        const float scale = hd < H ? q_scale : k_scale;
        const T* x = row + (size_t)hd * D;
        float* o = out + (size_t)hd * Dp;
        if (u < rot_pairs) {
            const int e0 = interleaved ? 2 * u : u, e1 = interleaved ? 2 * u + 1 : u + rot_pairs;
            const float a = ns_ld(x, e0), b = ns_ld(x, e1);
            float sn, cs;
            sincosf(fpos * inv_freq[u], &sn, &cs);
            sn *= magnitude; cs *= magnitude;
            o[e0] = (a * cs - b * sn) * scale;
            o[e1] = (b * cs + a * sn) * scale;
        } else {
            const int e = 2 * rot_pairs + (u - rot_pairs);
            o[e] = e < D ? ns_ld(x, e) * scale : 0.f;
        }
    }
    float* ov = out + (size_t)2 * H * Dp;
    for (int e = threadIdx.x; e < H * V; e += blockDim.x) ov[e] = ns_ld(row, (size_t)2 * H * D + e);
    __syncthreads();  // the rotated rows are complete
    const int lane = threadIdx.x & 31;
    for (int hd = threadIdx.x >> 5; hd < H; hd += blockDim.x >> 5) {
        float qk = 0.f;
        for (int e = lane; e < D; e += 32) qk = fmaf(out[(size_t)hd * Dp + e], out[(size_t)(H + hd) * Dp + e], qk);
        qk = ns_warp_sum(qk);
        if (lane == 0) ov[H * V + hd] = qk;
    }
}

// ---------------------------------------------------------------------------------------
// the scan.  grid (request, head, columns / COLS); 128 threads.  A column of S is held by LPC lanes (4, 8 or 16) of one
// warp, R = Dp / LPC rows each: lane = part * (32 / LPC) + column, part p holds rows p*R .. p*R + R - 1.  The operands
// of 16 tokens at a time (8 for the widest heads) are brought to shared memory with cp.async, two stages deep, so the
// walk over the tokens waits for memory once per stage and not once per token; a row of q or k lies there in LPC
// segments of R + 4 floats (the parts' 16-byte reads then fall into different banks).
// q and k heads are shared by H / G heads each.  gate: per token and head (row stride ld) or null, then `decay[h]` is
// used; beta: null selects the plain rule.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int R>
__device__ __forceinline__ void load_row(const float* p, float (&x)[R]) {
#pragma unroll
    for (int i = 0; i < R / 4; ++i) {
        const float4 f = reinterpret_cast<const float4*>(p)[i];
        x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
    }
}

template <int R>
__device__ __forceinline__ float dot_part(const float (&s)[R], const float (&x)[R]) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;  // four partial sums, always combined in the same order
#pragma unroll
    for (int i = 0; i < R; i += 4) {
        a0 = fmaf(s[i], x[i], a0); a1 = fmaf(s[i + 1], x[i + 1], a1);
        a2 = fmaf(s[i + 2], x[i + 2], a2); a3 = fmaf(s[i + 3], x[i + 3], a3);
    }
    return (a0 + a1) + (a2 + a3);
}
template <int LPC>
__device__ __forceinline__ float sum_parts(float v) {  // over the LPC lanes of a column
#pragma unroll
    for (int off = 32 / LPC; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

template <int R, int LPC, int C, bool ONE>
struct ScanShape {
    static constexpr int kCols = C * 128 / LPC;             // columns per block
    static constexpr int kDp = R * LPC;
    // tokens per stage; ONE: a step in which every request brings one token keeps its blocks small, so that many of them
    // fit an SM and the state, which is all that such a step moves, streams at full rate
    static constexpr int kTokens = ONE ? 1 : (kDp > 128 ? 8 : 16);
    static constexpr int kSeg = R + 4, kRow = LPC * kSeg;   // a staged row of q or k
    static constexpr int kStage = kTokens * (2 * kRow + kCols + 4);  // floats: q rows, k rows, v slices, gates, betas, k . q
    static constexpr size_t kBytes = 2 * (size_t)kStage * sizeof(float);
};

// C columns per lane (their sums are independent of one another); the launcher uses 1.
template <int R, int LPC, int C, bool ONE>
__global__ void __launch_bounds__(128)
linear_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const float* __restrict__ gate, const float* __restrict__ beta, const float* __restrict__ kq,
                   const float* __restrict__ decay, int ld, float* __restrict__ state, long long state_floats,
                   const int* __restrict__ qo_indptr, const int* __restrict__ state_slot, float* __restrict__ out, int ld_out,
                   int H, int G, int D, int V) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    using Sh = ScanShape<R, LPC, C, ONE>;
    constexpr int CW = 32 / LPC;       // columns per warp and turn
    constexpr int CB = 128 / LPC;      // columns per block and turn
    extern __shared__ __align__(16) float scan_smem[];
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = lane / CW;
    const int col = warp * CW + (lane % CW);       // this lane's first column within the block; the others follow CB apart
    const int e0 = blockIdx.z * Sh::kCols;
    const int start = qo_indptr[b], end = qo_indptr[b + 1];
    if (end <= start) return;
    const int hk = h / (H / G);
    float* S_mem = state + (long long)state_slot[b] * state_floats + ((long long)h * D + part * R) * V + e0 + col;
    bool active[C];
    float S[C][R];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        active[c] = e0 + col + c * CB < V;
#pragma unroll
        for (int r = 0; r < R; ++r) S[c][r] = (active[c] && part * R + r < D) ? S_mem[(size_t)r * V + c * CB] : 0.f;
    }
    const float fixed = decay ? decay[h] : 1.f;
    const float* qh = q + (size_t)hk * Sh::kDp;
    const float* kh = k + (size_t)hk * Sh::kDp;
    const float* vh = v + (size_t)h * V + e0;
    const int n_cols = min(Sh::kCols, V - e0);

    auto issue = [&](int chunk) {  // the operands of tokens chunk*kTokens .. of this request into stage chunk & 1
        float* st = scan_smem + (size_t)(chunk & 1) * Sh::kStage;
        const int n0 = start + chunk * Sh::kTokens, cnt = min(Sh::kTokens, end - n0);
        constexpr int kPieces = Sh::kDp / 4;  // 16-byte pieces of a row
        for (int i = tid; i < cnt * kPieces; i += 128) {
            const int t = i / kPieces, j = i - t * kPieces;
            const int p = (4 * j) / R, within = 4 * j - p * R;
            cp_async16(st + t * Sh::kRow + p * Sh::kSeg + within, qh + (size_t)(n0 + t) * ld + 4 * j);
            cp_async16(st + Sh::kTokens * Sh::kRow + t * Sh::kRow + p * Sh::kSeg + within, kh + (size_t)(n0 + t) * ld + 4 * j);
        }
        float* sv = st + 2 * Sh::kTokens * Sh::kRow;
        for (int i = tid; i < cnt * n_cols; i += 128) {
            const int t = i / n_cols, c = i - t * n_cols;
            cp_async4(sv + t * Sh::kCols + c, vh + (size_t)(n0 + t) * ld + c);
        }
        float* sg = sv + Sh::kTokens * Sh::kCols;
        if (tid < cnt) {
            if (gate) cp_async4(sg + tid, gate + (size_t)(n0 + tid) * ld + h);
            if (beta) cp_async4(sg + Sh::kTokens + tid, beta + (size_t)(n0 + tid) * ld + h);
            cp_async4(sg + 2 * Sh::kTokens + tid, kq + (size_t)(n0 + tid) * ld + hk);
        }
    };

    const int n_chunks = (end - start + Sh::kTokens - 1) / Sh::kTokens;
    issue(0);
    cp_async_commit();
    for (int ch = 0; ch < n_chunks; ++ch) {
        if (ch + 1 < n_chunks) issue(ch + 1);
        cp_async_commit();
        cp_async_wait<1>();  // stage ch has landed (the group after it may still travel)
        __syncthreads();
        const float* st = scan_smem + (size_t)(ch & 1) * Sh::kStage;
        const float* sv = st + 2 * Sh::kTokens * Sh::kRow;
        const float* sg = sv + Sh::kTokens * Sh::kCols;
        const int n0 = start + ch * Sh::kTokens, cnt = min(Sh::kTokens, end - n0);
        // the operands of the next token are read from shared memory while this one's sums travel through the shuffles
        // (the widest heads would not keep two tokens' operands in registers)
        constexpr bool kAhead = R <= 32 && !ONE;
        constexpr int RN = kAhead ? R : 4;
        float kn[RN], qn[RN];
        if (kAhead) {
            load_row<RN>(st + Sh::kTokens * Sh::kRow + part * Sh::kSeg, kn);
            load_row<RN>(st + part * Sh::kSeg, qn);
        }
        for (int t = 0; t < cnt; ++t) {
            float kc[R], qc[R];
            if (kAhead) {
#pragma unroll
                for (int r = 0; r < R; ++r) { kc[r] = kn[r % RN]; qc[r] = qn[r % RN]; }
                if (t + 1 < cnt) {
                    load_row<RN>(st + Sh::kTokens * Sh::kRow + (t + 1) * Sh::kRow + part * Sh::kSeg, kn);
                    load_row<RN>(st + (t + 1) * Sh::kRow + part * Sh::kSeg, qn);
                }
            } else {
                load_row<R>(st + Sh::kTokens * Sh::kRow + t * Sh::kRow + part * Sh::kSeg, kc);
                load_row<R>(st + t * Sh::kRow + part * Sh::kSeg, qc);
            }
            const float gc = gate ? sg[t] : fixed;
            const float kqc = sg[2 * Sh::kTokens + t];
            const float bc = beta ? sg[Sh::kTokens + t] : 0.f;
            // both sums over a column from the state as the last token left it, side by side, for all of the lane's columns
            float dq[C], dk[C], w[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                w[c] = sv[t * Sh::kCols + col + c * CB];
                dq[c] = dot_part<R>(S[c], qc);
                dk[c] = beta ? dot_part<R>(S[c], kc) : 0.f;
            }
#pragma unroll
            for (int off = 32 / LPC; off < 32; off <<= 1) {
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    if (beta) dk[c] += __shfl_xor_sync(0xffffffffu, dk[c], off);
                    dq[c] += __shfl_xor_sync(0xffffffffu, dq[c], off);
                }
            }
#pragma unroll
            for (int c = 0; c < C; ++c) {
                if (beta) w[c] = bc * (w[c] - gc * dk[c]);
#pragma unroll
                for (int r = 0; r < R; ++r) S[c][r] = fmaf(kc[r], w[c], gc * S[c][r]);
                const float o = fmaf(w[c], kqc, gc * dq[c]);
                if (active[c] && part == 0) out[(size_t)(n0 + t) * ld_out + h * V + e0 + col + c * CB] = o;
            }
        }
        __syncthreads();  // the stage may be refilled
    }
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (active[c] && part * R + r < D) S_mem[(size_t)r * V + c * CB] = S[c][r];
}

// ---------------------------------------------------------------------------------------
// read-out to mixer output: per (token, head) o / sqrt(mean(o^2) + eps) * gain[e] (gain may be null)
// * silu(gate[token, h*V + e]); one warp per (token, head), rounded once to T.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, int ld_o, const T* __restrict__ gate, int ld_gate,
                                      const float* __restrict__ gain, float eps, T* __restrict__ out, int ld_out,
                                      const int* __restrict__ token_req, int n_tokens, int H, int V) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)n_tokens * H) return;
    const int n = (int)(w / H), h = (int)(w % H), lane = threadIdx.x & 31;
    if (token_req[n] < 0) return;
    const float* x = o + (size_t)n * ld_o + (size_t)h * V;
    float ss = 0.f;
    for (int e = lane; e < V; e += 32) ss += x[e] * x[e];
    const float inv = rsqrtf(ns_warp_sum(ss) / (float)V + eps);
    for (int e = lane; e < V; e += 32) {
        float y = x[e] * inv;
        if (gain) y *= gain[e];
        if (gate) y *= silu_f(ns_ld(gate, (size_t)n * ld_gate + (size_t)h * V + e));
        ns_st(out, (size_t)n * ld_out + (size_t)h * V + e, y);
    }
}

}  // namespace

NS_API int ns_delta_prepare(const void* proj, int ld_proj, const float* taps, int n_taps, const float* a_log, const float* dt_bias,
                            float* state, long long state_floats, long long tail_off, const int* token_req, const int* qo_indptr,
                            const int* state_slot, float* rec, int ld_rec, int n_tokens, int n_requests, int G, int H, int D, int Dp,
                            int V, int off_b, int off_a, float q_scale, float unit_eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (n_taps < 1 || G < 1 || H % G || Dp < D || Dp % 4) NS_FAIL(NS_ERR_ARGUMENT, "ns_delta_prepare: taps=%d heads=%d/%d D=%d Dp=%d", n_taps, H, G, D, Dp);
    const int C = 2 * G * D + H * V;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_delta_prepare: %d channels do not fit shared memory", C);
    if (dtype != NS_F32 && dtype != NS_BF16) NS_FAIL(NS_ERR_ARGUMENT, "ns_delta_prepare: unknown dtype %d", dtype);
    if (smem > 48 * 1024) {
        if (dtype == NS_F32) NS_CUDA(cudaFuncSetAttribute(delta_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        else NS_CUDA(cudaFuncSetAttribute(delta_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    const dim3 tail_grid(n_requests, (C + 255) / 256);
    if (dtype == NS_F32) {
        NS_LAUNCH((delta_prepare_kernel<float>), n_tokens, 256, smem, stream, (const float*)proj, ld_proj, taps, n_taps, a_log, dt_bias,
                  state, state_floats, tail_off, token_req, qo_indptr, state_slot, rec, ld_rec, G, H, D, Dp, V, off_b, off_a, q_scale, unit_eps);
        if (n_taps > 1)
            NS_LAUNCH((conv_tail_kernel<float>), tail_grid, 256, 0, stream, (const float*)proj, ld_proj, state, state_floats, tail_off,
                      qo_indptr, state_slot, C, n_taps);
    } else {
        NS_LAUNCH((delta_prepare_kernel<__nv_bfloat16>), n_tokens, 256, smem, stream, (const __nv_bfloat16*)proj, ld_proj, taps, n_taps, a_log,
                  dt_bias, state, state_floats, tail_off, token_req, qo_indptr, state_slot, rec, ld_rec, G, H, D, Dp, V, off_b, off_a, q_scale, unit_eps);
        if (n_taps > 1)
            NS_LAUNCH((conv_tail_kernel<__nv_bfloat16>), tail_grid, 256, 0, stream, (const __nv_bfloat16*)proj, ld_proj, state, state_floats,
                      tail_off, qo_indptr, state_slot, C, n_taps);
    }
    NS_CHECK_LAUNCH("ns_delta_prepare");
    return NS_OK;
}

// The tail's move alone, for a mixer that runs a short convolution over the leading C channels of its projection in a
// kernel of its own: after that kernel, every request's last n_taps - 1 inputs (in `state` at `tail_off`) move on by this
// step's tokens.
NS_API int ns_conv_tail(const void* proj, int ld_proj, float* state, long long state_floats, long long tail_off, const int* qo_indptr,
                        const int* state_slot, int C, int n_taps, int n_requests, int dtype, cudaStream_t stream) {
    if (n_requests <= 0 || n_taps <= 1 || C <= 0) return NS_OK;
    const dim3 grid(n_requests, (C + 255) / 256);
    if (dtype == NS_F32)
        NS_LAUNCH((conv_tail_kernel<float>), grid, 256, 0, stream, (const float*)proj, ld_proj, state, state_floats, tail_off, qo_indptr,
                  state_slot, C, n_taps);
    else if (dtype == NS_BF16)
        NS_LAUNCH((conv_tail_kernel<__nv_bfloat16>), grid, 256, 0, stream, (const __nv_bfloat16*)proj, ld_proj, state, state_floats,
                  tail_off, qo_indptr, state_slot, C, n_taps);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_conv_tail: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_conv_tail");
    return NS_OK;
}

NS_API int ns_rotary_prepare(const void* proj, int ld_proj, const int* positions, const int* token_req, const float* inv_freq,
                             float magnitude, int interleaved, int rot_pairs, float* rec, int ld_rec, int n_tokens, int H, int D,
                             int Dp, int V, float q_scale, float k_scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (rot_pairs < 0 || 2 * rot_pairs > D || Dp < D || Dp % 4) NS_FAIL(NS_ERR_ARGUMENT, "ns_rotary_prepare: %d pairs, D=%d, Dp=%d", rot_pairs, D, Dp);
    if (dtype == NS_F32)
        NS_LAUNCH((rotary_prepare_kernel<float>), n_tokens, 256, 0, stream, (const float*)proj, ld_proj, positions, token_req, inv_freq,
                  magnitude, interleaved, rot_pairs, rec, ld_rec, H, D, Dp, V, q_scale, k_scale);
    else if (dtype == NS_BF16)
        NS_LAUNCH((rotary_prepare_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, (const __nv_bfloat16*)proj, ld_proj, positions, token_req,
                  inv_freq, magnitude, interleaved, rot_pairs, rec, ld_rec, H, D, Dp, V, q_scale, k_scale);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_rotary_prepare: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_rotary_prepare");
    return NS_OK;
}

// The width that the scan pads a head of D features to: the smallest of 16, 32, 64, 128, 256 that holds it.
NS_API int ns_linear_scan_rows(int D) {
    for (int r : {4, 8, 16, 32, 64})
        if (4 * r >= D) return r;
    return 0;
}

namespace {
template <int R, int LPC, int C, bool ONE>
int launch_scan_as(const float* q, const float* k, const float* v, const float* gate, const float* beta, const float* kq,
                const float* decay, int ld, float* state, long long state_floats, const int* qo_indptr, const int* state_slot, float* out, int ld_out,
                int n_requests, int H, int G, int D, int V, cudaStream_t stream) {
    using Sh = ScanShape<R, LPC, C, ONE>;
    static bool configured = false;
    if (!configured && Sh::kBytes > 48 * 1024) {
        NS_CUDA(cudaFuncSetAttribute(linear_scan_kernel<R, LPC, C, ONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sh::kBytes));
        configured = true;
    }
    const int col_blocks = (V + Sh::kCols - 1) / Sh::kCols;
    if (H > 65535 || col_blocks > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_linear_scan: %d heads of %d columns exceed the grid", H, V);
    NS_LAUNCH((linear_scan_kernel<R, LPC, C, ONE>), dim3(n_requests, H, col_blocks), 128, Sh::kBytes, stream, q, k, v, gate, beta, kq, decay, ld,
              state, state_floats, qo_indptr, state_slot, out, ld_out, H, G, D, V);
    NS_CHECK_LAUNCH("ns_linear_scan");
    return NS_OK;
}

template <int R, int LPC, int C>
int launch_scan(const float* q, const float* k, const float* v, const float* gate, const float* beta, const float* kq,
                const float* decay, int ld, float* state, long long state_floats, const int* qo_indptr, const int* state_slot,
                float* out, int ld_out, int n_requests, int H, int G, int D, int V, cudaStream_t stream, int longest) {
    if (longest <= 1)
        return launch_scan_as<R, LPC, C, true>(q, k, v, gate, beta, kq, decay, ld, state, state_floats, qo_indptr, state_slot, out,
                                               ld_out, n_requests, H, G, D, V, stream);
    return launch_scan_as<R, LPC, C, false>(q, k, v, gate, beta, kq, decay, ld, state, state_floats, qo_indptr, state_slot, out,
                                            ld_out, n_requests, H, G, D, V, stream);
}
}  // namespace

namespace { int g_scan_lanes = 0; }
// 0 (default): the launcher chooses the lanes per column; 4 or 8 force a choice (for measurements).
NS_API int ns_linear_scan_lanes(int lanes) {
    g_scan_lanes = lanes;
    return NS_OK;
}

// `longest`: the most tokens any request brings to this step (1 for decoding).  Long walks over few columns take eight lanes
// per column instead of four: twice the blocks and half the work per token and lane.
NS_API int ns_linear_scan(const float* q, const float* k, const float* v, const float* gate, const float* beta, const float* kq,
                          const float* decay, int ld, float* state, long long state_floats, const int* qo_indptr, const int* state_slot, float* out,
                          int ld_out, int n_requests, int H, int G, int D, int V, int longest, int n_sms, cudaStream_t stream) {
    if (n_requests <= 0) return NS_OK;
    const int R4 = ns_linear_scan_rows(D);
    if (!R4) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_linear_scan: a head of %d features (at most 256)", D);
    if (G < 1 || H % G) NS_FAIL(NS_ERR_ARGUMENT, "ns_linear_scan: %d heads over %d key heads", H, G);
    if (!gate && !decay) NS_FAIL(NS_ERR_ARGUMENT, "ns_linear_scan: neither a gate per token nor a decay per head");
    if (!kq) NS_FAIL(NS_ERR_ARGUMENT, "ns_linear_scan: no k . q per token");
    if (ld % 4 || ((uintptr_t)q | (uintptr_t)k) % 16) NS_FAIL(NS_ERR_ARGUMENT, "ns_linear_scan: q and k rows must be 16-byte aligned");
    // Many tokens to walk and few columns to walk them on: eight lanes per column, whose sums per lane are half as long
    // (measured on a B200, 2,048 tokens of one request, 16 heads of 128 x 128: 0.43 us per token with four lanes, 0.34 with
    // eight, 0.44 with sixteen and two columns per lane - the shuffles then outweigh the shorter sums); otherwise four,
    // which read and write the state in whole sectors.
    const long long blocks4 = (long long)n_requests * H * ((V + 31) / 32);
    const int sms = n_sms > 0 ? n_sms : 148;
    const int lanes = g_scan_lanes == 4 || g_scan_lanes == 8 ? g_scan_lanes : (longest >= 64 && R4 >= 8 && blocks4 < 4ll * sms ? 8 : 4);
#define NS_SCAN_ARGS q, k, v, gate, beta, kq, decay, ld, state, state_floats, qo_indptr, state_slot, out, ld_out, n_requests, H, G, D, V, stream, longest
    switch (R4) {
        case 4: return launch_scan<4, 4, 1>(NS_SCAN_ARGS);
        case 8: return lanes == 8 ? launch_scan<4, 8, 1>(NS_SCAN_ARGS) : launch_scan<8, 4, 1>(NS_SCAN_ARGS);
        case 16: return lanes == 8 ? launch_scan<8, 8, 1>(NS_SCAN_ARGS) : launch_scan<16, 4, 1>(NS_SCAN_ARGS);
        case 32: return lanes == 8 ? launch_scan<16, 8, 1>(NS_SCAN_ARGS) : launch_scan<32, 4, 1>(NS_SCAN_ARGS);
        case 64: return lanes == 8 ? launch_scan<32, 8, 1>(NS_SCAN_ARGS) : launch_scan<64, 4, 1>(NS_SCAN_ARGS);
    }
#undef NS_SCAN_ARGS
    NS_FAIL(NS_ERR_UNSUPPORTED, "ns_linear_scan: head of %d features", D);
}

NS_API int ns_head_norm_gate(const float* o, int ld_o, const void* gate, int ld_gate, const float* gain, float eps, void* out,
                             int ld_out, const int* token_req, int n_tokens, int H, int V, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    const long long warps = (long long)n_tokens * H;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (dtype == NS_F32)
        NS_LAUNCH((head_norm_gate_kernel<float>), blocks, 128, 0, stream, o, ld_o, (const float*)gate, ld_gate, gain, eps, (float*)out,
                  ld_out, token_req, n_tokens, H, V);
    else if (dtype == NS_BF16)
        NS_LAUNCH((head_norm_gate_kernel<__nv_bfloat16>), blocks, 128, 0, stream, o, ld_o, (const __nv_bfloat16*)gate, ld_gate, gain, eps,
                  (__nv_bfloat16*)out, ld_out, token_req, n_tokens, H, V);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_head_norm_gate: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_head_norm_gate");
    return NS_OK;
}
