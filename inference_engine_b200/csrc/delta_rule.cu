// Kernels of the gated delta rule mixer with one decay per head and key channel.
//
// A request's state slot holds, in 32-bit floats: per head the matrix S (dim x vdim), stored
// column by column ([heads][vdim][dim]), then the last taps - 1 inputs of the short convolutions
// ([taps - 1][channels], oldest first).
//
//  * delta_prep: per token the short causal convolution (per channel, over the step's earlier
//    tokens of the same request and, before them, the slot's kept inputs) and silu of q, k, v;
//    q and k as unit vectors per head (q also times dim^-1/2); beta = sigmoid(.); the decay
//    g = exp(-exp(A_log[head]) * softplus(a + dt_bias)).
//  * delta_conv_tail: the slot's kept inputs moved on by the step's tokens.
//  * delta_rule: per token, in order:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;
//    o = S^T q.  Columns of S do not interact: a block owns some columns of one head of one
//    request, a group of TPC lanes one column (lane j of the group holds rows R j .. R j + R - 1),
//    and walks the request's tokens of this step in order, eight at a time through shared memory.
//    Each sum over rows is taken in an order that depends on `dim` alone.
//  * gated_rms_heads: o / rms(o) per head, times a weight, times sigmoid(gate).
// Everything here is 32-bit.
#include "common.cuh"
#include <math.h>

namespace {

__device__ __forceinline__ float silu_f(float y) { return y / (1.0f + expf(-y)); }
__device__ __forceinline__ float sigmoid_f(float y) { return 1.0f / (1.0f + expf(-y)); }
__device__ __forceinline__ float softplus_f(float y) { return y > 20.0f ? y : log1pf(expf(y)); }

// grid: (tokens, units).  The units of a token: the q heads, the k heads (convolution, silu, unit
// norm over `dim` channels each), the v heads (convolution and silu over `vdim` channels each), the
// heads' decays (`dim` values each), and one unit for the betas.  channels = 2 * kv_heads * dim +
// heads * vdim; qkvb rows hold the channels and then `heads` betas.
__device__ __forceinline__ void
delta_prep_unit(int n, int unit, float* y, float* red,
                const float* __restrict__ qkvb, int ld, const float* __restrict__ a,
                  const float* __restrict__ conv_w, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, const float* __restrict__ state, long long state_stride,
                  const int* __restrict__ slots, const int* __restrict__ seq_of_token,
                  const int* __restrict__ cu_q, float* __restrict__ q_out, float* __restrict__ k_out,
                  float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay,
                  int heads, int kv_heads, int dim, int vdim, int taps, int num_slots, int* err) {
    int tid = threadIdx.x;
    int qk = kv_heads * dim, channels = 2 * qk + heads * vdim;
    if (unit == 2 * kv_heads + 2 * heads) {  // the betas
        for (int h = tid; h < heads; h += blockDim.x) beta[(size_t)n * heads + h] = sigmoid_f(qkvb[(size_t)n * ld + channels + h]);
        return;
    }
    if (unit >= 2 * kv_heads + heads) {  // a head's decays
        int h = unit - 2 * kv_heads - heads;
        float rate = expf(A_log[h]);
        for (int d = tid; d < dim; d += blockDim.x) {
            size_t i = (size_t)n * heads * dim + h * dim + d;
            decay[i] = expf(-rate * softplus_f(a[i] + dt_bias[h * dim + d]));
        }
        return;
    }
    int seq = seq_of_token[n];
    int t = n - cu_q[seq];  // the token's place among the request's tokens of this step
    int slot = slots[seq];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) ie_report(err, IE_ERR_PAGE, slot, n);
        return;
    }
    bool is_v = unit >= 2 * kv_heads;
    int width = is_v ? vdim : dim;
    int first = is_v ? 2 * qk + (unit - 2 * kv_heads) * vdim : unit * dim;  // the unit's first channel
    const float* tail = state + (size_t)slot * state_stride + (size_t)heads * dim * vdim;
    float ss = 0.f;
    for (int i = tid; i < width; i += blockDim.x) {
        int c = first + i;
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            int back = taps - 1 - j;  // this tap looks `back` tokens back
            float x = (t - back >= 0) ? qkvb[(size_t)(n - back) * ld + c]
                                      : tail[(size_t)(taps - 1 + t - back) * channels + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        float sv = silu_f(acc);
        if (is_v) v_out[(size_t)n * heads * vdim + (c - 2 * qk)] = sv;
        else { y[i] = sv; ss = fmaf(sv, sv, ss); }
    }
    if (is_v) return;
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float f = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) + 1e-6f);
    bool is_q = unit < kv_heads;
    if (is_q) f *= 1.0f / sqrtf((float)dim);
    float* dst = (is_q ? q_out : k_out) + (size_t)n * qk + (is_q ? unit : unit - kv_heads) * dim;
    for (int i = tid; i < dim; i += blockDim.x) dst[i] = y[i] * f;
    __syncthreads();  // (y and red are used again by the block's next unit)
}

// grid: (tokens, blocks per token); a block takes the token's units blockIdx.y, blockIdx.y + gridDim.y, ...
// (a block per unit when the step has few tokens, a few blocks per token when it has many).
__global__ void __launch_bounds__(128)
delta_prep_kernel(const float* __restrict__ qkvb, int ld, const float* __restrict__ a,
                  const float* __restrict__ conv_w, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, const float* __restrict__ state, long long state_stride,
                  const int* __restrict__ slots, const int* __restrict__ seq_of_token,
                  const int* __restrict__ cu_q, float* __restrict__ q_out, float* __restrict__ k_out,
                  float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay,
                  int heads, int kv_heads, int dim, int vdim, int taps, int num_slots, int* err) {
    extern __shared__ float y[];  // [max(dim, vdim)]: one unit's channels after the convolution
    __shared__ float red[4];
    ie_pdl_trigger();
    ie_pdl_wait();
    int units = 2 * kv_heads + 2 * heads + 1;
    for (int unit = blockIdx.y; unit < units; unit += gridDim.y)
        delta_prep_unit(blockIdx.x, unit, y, red, qkvb, ld, a, conv_w, A_log, dt_bias, state, state_stride, slots,
                        seq_of_token, cu_q, q_out, k_out, v_out, beta, decay, heads, kv_heads, dim, vdim, taps,
                        num_slots, err);
}

// One block per request of the step: the kept inputs become the last taps - 1 of (kept, new).
__global__ void delta_conv_tail_kernel(const float* __restrict__ qkvb, int ld, float* __restrict__ state,
                                       long long state_stride, const int* __restrict__ slots,
                                       const int* __restrict__ cu_q, long long matrix_floats, int channels,
                                       int taps, int num_slots) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int seq = blockIdx.x;
    int start = cu_q[seq], len = cu_q[seq + 1] - start;
    int slot = slots[seq];
    if (len <= 0 || slot < 0 || slot >= num_slots) return;
    float* tail = state + (size_t)slot * state_stride + matrix_floats;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        // row j takes the input at step-relative time len - (taps - 1) + j; a thread owns a channel and
        // goes through the rows in rising order, so a kept row is read before it is overwritten
        for (int j = 0; j < taps - 1; ++j) {
            int tt = len - (taps - 1) + j;
            float x = tt >= 0 ? qkvb[(size_t)(start + tt) * ld + c] : tail[(size_t)(taps - 1 + tt) * channels + c];
            tail[(size_t)j * channels + c] = x;
        }
    }
}

constexpr int DR_THREADS = 128;
constexpr int DR_CHUNK = 8;  // tokens staged in shared memory at a time

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async16f(float* dst, const float* src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// grid: (column blocks, heads, requests).  R rows per lane; TPC lanes per column (a power of two).
// The tokens' k, q, decay, v and beta come through shared memory eight tokens at a time, the next
// eight on their way (cp.async, two buffers) while these are worked on.  A lane holds R (8 or 16)
// consecutive rows of its column; in shared memory a token's k, q and decay lie in groups of R
// entries R + 4 floats apart, so that a lane fetches its rows with 16-byte loads and the lanes of a
// column hit different banks; entries beyond `dim` read as zero, so the inner loops carry no bounds checks.
template <int R, int TPC>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                  float* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int num_slots) {
    extern __shared__ __align__(16) float sm[];  // two buffers of: k, q, g [CHUNK][DP] each, v [CHUNK][COLS], beta [CHUNK]
    static_assert(R == 8 || R == 16, "a lane's rows are one group of 8 or 16");
    constexpr int GS = R + 4;  // a lane's group of R entries, and four floats to the next lane's
    constexpr int COLS = DR_THREADS / TPC, DP = GS * TPC;  // a token's row of k (q, decay)
    constexpr int BUF = DR_CHUNK * (3 * DP + COLS + 4);
    ie_pdl_trigger();
    ie_pdl_wait();
    int seq = blockIdx.z, head = blockIdx.y;
    int start = cu_q[seq], len = cu_q[seq + 1] - start;
    int slot = slots[seq];
    if (len <= 0 || slot < 0 || slot >= num_slots) return;
    int tid = threadIdx.x;
    int sub = tid % TPC, my_col = tid / TPC, col = blockIdx.x * COLS + my_col;
    bool live = col < vdim;
    int kvh = head / (heads / kv_heads);
    float* S = state + (size_t)slot * state_stride + ((size_t)head * vdim + (live ? col : 0)) * dim;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        int r = sub * R + i;
        s[i] = (live && r < dim) ? S[r] : 0.f;
    }
    // what the copies never touch (entries beyond dim, the gaps) reads as zero
    for (int i = tid; i < 2 * BUF; i += DR_THREADS) sm[i] = 0.f;
    __syncthreads();
    int c0 = blockIdx.x * COLS;
    bool vec = (dim % 4 == 0) && (vdim % 4 == 0) && (COLS % 4 == 0);
    auto stage = [&](int t0, int b) {  // the chunk's values on their way into buffer b
        int cnt = min(DR_CHUNK, len - t0);
        float* ks = sm + b * BUF;
        float* qs = ks + DR_CHUNK * DP;
        float* gs = qs + DR_CHUNK * DP;
        float* vs = gs + DR_CHUNK * DP;
        float* bs = vs + DR_CHUNK * COLS;
        if (vec) {  // rows and column runs of whole 16-byte pieces
            int dq = dim >> 2;
            for (int i = tid; i < cnt * dq; i += DR_THREADS) {
                int tt = i / dq, d = (i - tt * dq) * 4;
                size_t n = (size_t)(start + t0 + tt);
                int at = tt * DP + (d / R) * GS + (d % R);
                cp_async16f(ks + at, k + (n * kv_heads + kvh) * dim + d);
                cp_async16f(qs + at, q + (n * kv_heads + kvh) * dim + d);
                cp_async16f(gs + at, decay + (n * heads + head) * dim + d);
            }
            for (int i = tid; i < cnt * (COLS / 4); i += DR_THREADS) {
                int tt = i / (COLS / 4), c = (i % (COLS / 4)) * 4;
                if (c0 + c < vdim) cp_async16f(vs + tt * COLS + c, v + ((size_t)(start + t0 + tt) * heads + head) * vdim + c0 + c);
            }
        } else {
            for (int tt = 0; tt < cnt; ++tt) {
                size_t n = (size_t)(start + t0 + tt);
                for (int d = tid; d < dim; d += DR_THREADS) {
                    int at = tt * DP + (d / R) * GS + (d % R);
                    cp_async4(ks + at, k + (n * kv_heads + kvh) * dim + d);
                    cp_async4(qs + at, q + (n * kv_heads + kvh) * dim + d);
                    cp_async4(gs + at, decay + (n * heads + head) * dim + d);
                }
                if (tid < COLS && c0 + tid < vdim) cp_async4(vs + tt * COLS + tid, v + (n * heads + head) * vdim + c0 + tid);
            }
        }
        if (tid < cnt) cp_async4(bs + tid, beta + (size_t)(start + t0 + tid) * heads + head);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    int b = 0;
    for (int t0 = 0; t0 < len; t0 += DR_CHUNK, b ^= 1) {
        int cnt = min(DR_CHUNK, len - t0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this chunk has landed for everyone, and everyone is done with the other buffer
        if (t0 + DR_CHUNK < len) stage(t0 + DR_CHUNK, b ^ 1);
        const float* ks = sm + b * BUF + sub * GS;
        const float* qs = ks + DR_CHUNK * DP;
        const float* gs = qs + DR_CHUNK * DP;
        const float* vs = sm + b * BUF + 3 * DR_CHUNK * DP + my_col;
        const float* bs = sm + b * BUF + 3 * DR_CHUNK * DP + DR_CHUNK * COLS;
        for (int tt = 0; tt < cnt; ++tt) {
            const float* kt = ks + tt * DP;
            const float* qt = qs + tt * DP;
            const float* gt = gs + tt * DP;
            float kv[R], gv[R], qv[R];
#pragma unroll
            for (int j = 0; j < R / 4; ++j) {
                *reinterpret_cast<float4*>(kv + 4 * j) = reinterpret_cast<const float4*>(kt)[j];
                *reinterpret_cast<float4*>(gv + 4 * j) = reinterpret_cast<const float4*>(gt)[j];
                *reinterpret_cast<float4*>(qv + 4 * j) = reinterpret_cast<const float4*>(qt)[j];
            }
            float d4[4] = {0.f, 0.f, 0.f, 0.f};  // four partial sums: shorter chains, a fixed order
#pragma unroll
            for (int i = 0; i < R; ++i) {
                s[i] *= gv[i];
                d4[i & 3] = fmaf(s[i], kv[i], d4[i & 3]);
            }
            float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
            for (int o = TPC >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            float u = bs[tt] * ((live ? vs[tt * COLS] : 0.f) - dot);
            float r4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < R; ++i) {
                s[i] = fmaf(kv[i], u, s[i]);
                r4[i & 3] = fmaf(s[i], qv[i], r4[i & 3]);
            }
            float rd = (r4[0] + r4[1]) + (r4[2] + r4[3]);
#pragma unroll
            for (int o = TPC >> 1; o > 0; o >>= 1) rd += __shfl_xor_sync(0xffffffffu, rd, o);
            if (live && sub == 0) out[((size_t)(start + t0 + tt) * heads + head) * vdim + col] = rd;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            int r = sub * R + i;
            if (r < dim) S[r] = s[i];
        }
    }
}

// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
gated_rms_heads_kernel(const float* __restrict__ o, const float* __restrict__ weight, float eps,
                       const float* __restrict__ gate_pre, T* __restrict__ out, long long rows, int vdim) {
    ie_pdl_trigger();
    ie_pdl_wait();
    long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    const float* src = o + row * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int d = lane; d < vdim; d += 32)
        ie_store(out + row * vdim + d, src[d] * inv * weight[d] * sigmoid_f(gate_pre[row * vdim + d]));
}
}  // namespace

IE_API int ie_delta_prep(const float* qkvb, int ld, const float* a, const float* conv_w, const float* A_log,
                         const float* dt_bias, float* state, long long state_stride, const int* slots,
                         const int* seq_of_token, const int* cu_q, float* q_out, float* k_out, float* v_out,
                         float* beta, float* decay, int num_tokens, int num_seqs, int heads, int kv_heads,
                         int dim, int vdim, int taps, int num_slots, int* err, void* stream) {
    if (num_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    size_t smem = (size_t)(dim > vdim ? dim : vdim) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    int units = 2 * kv_heads + 2 * heads + 1;
    int per_token = num_tokens >= 512 ? (units < 4 ? units : 4) : units;
    int e = ie_launch(delta_prep_kernel, dim3(num_tokens, per_token), dim3(128), smem, s, qkvb, ld, a, conv_w, A_log, dt_bias,
                      (const float*)state, state_stride, slots, seq_of_token, cu_q, q_out, k_out, v_out, beta,
                      decay, heads, kv_heads, dim, vdim, taps, num_slots, err);
    if (e != 0 || taps < 2) return e;
    int channels = 2 * kv_heads * dim + heads * vdim;
    return ie_launch(delta_conv_tail_kernel, dim3(num_seqs), dim3(256), 0, s, qkvb, ld, state, state_stride, slots,
                     cu_q, (long long)heads * dim * vdim, channels, taps, num_slots);
}

template <int R, int TPC>
static int launch_delta_rule(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                             float* state, long long state_stride, const int* slots, const int* cu_q, float* out,
                             int num_seqs, int heads, int kv_heads, int dim, int vdim, int num_slots, cudaStream_t s) {
    constexpr int COLS = DR_THREADS / TPC;
    size_t smem = (size_t)2 * DR_CHUNK * (3 * (R + 4) * TPC + COLS + 4) * sizeof(float);
    static IePerDevice allowed;
    cudaError_t e = ie_allow_smem(allowed, delta_rule_kernel<R, TPC>, 160 * 1024);  // (dim 512: 124 KB)
    if (e != cudaSuccess) return (int)e;
    dim3 grid((vdim + COLS - 1) / COLS, heads, num_seqs);
    return ie_launch(delta_rule_kernel<R, TPC>, grid, dim3(DR_THREADS), smem, s, q, k, v, beta, decay, state,
                     state_stride, slots, cu_q, out, heads, kv_heads, dim, vdim, num_slots);
}

IE_API int ie_delta_rule(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                         float* state, long long state_stride, const int* slots, const int* cu_q, float* out,
                         int num_seqs, int heads, int kv_heads, int dim, int vdim, int num_slots, void* stream) {
    if (num_seqs <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
#define IE_DR_ARGS q, k, v, beta, decay, state, state_stride, slots, cu_q, out, num_seqs, heads, kv_heads, dim, vdim, num_slots, s
    // Eight rows per lane for small key sizes (2,048 tokens of 8 heads of 64 x 64: 0.54 ms against 0.65 with
    // sixteen), sixteen from there on (16 heads of 128 x 128: 0.64 ms against 0.75 with eight: the exchange
    // between a column's lanes has a step more).
    if (dim <= 8) return launch_delta_rule<8, 1>(IE_DR_ARGS);
    if (dim <= 16) return launch_delta_rule<8, 2>(IE_DR_ARGS);
    if (dim <= 32) return launch_delta_rule<8, 4>(IE_DR_ARGS);
    if (dim <= 64) return launch_delta_rule<8, 8>(IE_DR_ARGS);
    if (dim <= 128) return launch_delta_rule<16, 8>(IE_DR_ARGS);
    if (dim <= 256) return launch_delta_rule<16, 16>(IE_DR_ARGS);
    if (dim <= 512) return launch_delta_rule<16, 32>(IE_DR_ARGS);
#undef IE_DR_ARGS
    return (int)cudaErrorInvalidValue;  // dim <= 512
}

IE_API int ie_gated_rms_heads(const float* o, const float* weight, float eps, const float* gate_pre, void* out,
                              int out_dtype, long long rows, int vdim, void* stream) {
    if (rows <= 0) return 0;
    dim3 grid((unsigned)((rows + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_BF16)
        return ie_launch(gated_rms_heads_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, o, weight, eps, gate_pre,
                         (__nv_bfloat16*)out, rows, vdim);
    return ie_launch(gated_rms_heads_kernel<float>, grid, dim3(128), 0, s, o, weight, eps, gate_pre, (float*)out,
                     rows, vdim);
}
