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
//    request, a group of TPC lanes one column (lane j of the group holds rows j, j + TPC, ...),
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

// One block per token.  channels = 2 * kv_heads * dim + heads * vdim; qkvb rows hold the channels
// and then `heads` betas.
__global__ void __launch_bounds__(256)
delta_prep_kernel(const float* __restrict__ qkvb, int ld, const float* __restrict__ a,
                  const float* __restrict__ conv_w, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, const float* __restrict__ state, long long state_stride,
                  const int* __restrict__ slots, const int* __restrict__ seq_of_token,
                  const int* __restrict__ cu_q, float* __restrict__ q_out, float* __restrict__ k_out,
                  float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay,
                  int heads, int kv_heads, int dim, int vdim, int taps, int num_slots, int* err) {
    extern __shared__ float y[];  // [2 * kv_heads * dim]: q and k after the convolution
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x, tid = threadIdx.x;
    int seq = seq_of_token[n];
    int t = n - cu_q[seq];  // the token's place among the request's tokens of this step
    int slot = slots[seq];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) ie_report(err, IE_ERR_PAGE, slot, n);
        return;
    }
    int qk = kv_heads * dim, channels = 2 * qk + heads * vdim;
    const float* tail = state + (size_t)slot * state_stride + (size_t)heads * dim * vdim;
    for (int c = tid; c < channels; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            int back = taps - 1 - j;  // this tap looks `back` tokens back
            float x;
            if (t - back >= 0) x = qkvb[(size_t)(n - back) * ld + c];
            else x = tail[(size_t)(taps - 1 + t - back) * channels + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        float s = silu_f(acc);
        if (c < 2 * qk) y[c] = s;
        else v_out[(size_t)n * heads * vdim + (c - 2 * qk)] = s;
    }
    __syncthreads();
    int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    for (int hh = warp; hh < 2 * kv_heads; hh += warps) {  // q heads, then k heads
        const float* src = y + hh * dim;
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = warp_sum(ss);
        float f = 1.0f / sqrtf(ss + 1e-6f);
        bool is_q = hh < kv_heads;
        if (is_q) f *= 1.0f / sqrtf((float)dim);
        float* dst = (is_q ? q_out : k_out) + (size_t)n * qk + (is_q ? hh : hh - kv_heads) * dim;
        for (int d = lane; d < dim; d += 32) dst[d] = src[d] * f;
    }
    for (int h = tid; h < heads; h += blockDim.x) beta[(size_t)n * heads + h] = sigmoid_f(qkvb[(size_t)n * ld + channels + h]);
    for (int i = tid; i < heads * dim; i += blockDim.x) {
        float rate = expf(A_log[i / dim]);
        decay[(size_t)n * heads * dim + i] = expf(-rate * softplus_f(a[(size_t)n * heads * dim + i] + dt_bias[i]));
    }
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

// grid: (column blocks, heads, requests).  R rows per lane; TPC lanes per column (a power of two).
template <int R>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ slots, const int* __restrict__ cu_q,
                  float* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int tpc, int num_slots) {
    extern __shared__ float sm[];  // per staged token: k[dim], q[dim], g[dim]; then v and beta
    ie_pdl_trigger();
    ie_pdl_wait();
    int seq = blockIdx.z, head = blockIdx.y;
    int start = cu_q[seq], len = cu_q[seq + 1] - start;
    int slot = slots[seq];
    if (len <= 0 || slot < 0 || slot >= num_slots) return;
    int tid = threadIdx.x;
    int cols_per_block = DR_THREADS / tpc;
    int sub = tid % tpc, col = blockIdx.x * cols_per_block + tid / tpc;
    bool live = col < vdim;
    int kvh = head / (heads / kv_heads);
    float* S = state + (size_t)slot * state_stride + ((size_t)head * vdim + (live ? col : 0)) * dim;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        int r = sub + i * tpc;
        s[i] = (live && r < dim) ? S[r] : 0.f;
    }
    float* ks = sm;                          // [CHUNK][dim]
    float* qs = ks + DR_CHUNK * dim;         // [CHUNK][dim]
    float* gs = qs + DR_CHUNK * dim;         // [CHUNK][dim]
    float* vs = gs + DR_CHUNK * dim;         // [CHUNK][cols_per_block]
    float* bs = vs + DR_CHUNK * cols_per_block;  // [CHUNK]
    int c0 = blockIdx.x * cols_per_block;
    for (int t0 = 0; t0 < len; t0 += DR_CHUNK) {
        int cnt = min(DR_CHUNK, len - t0);
        __syncthreads();
        for (int i = tid; i < cnt * dim; i += DR_THREADS) {
            int tt = i / dim, d = i - tt * dim;
            size_t n = (size_t)(start + t0 + tt);
            ks[i] = k[(n * kv_heads + kvh) * dim + d];
            qs[i] = q[(n * kv_heads + kvh) * dim + d];
            gs[i] = decay[(n * heads + head) * dim + d];
        }
        for (int i = tid; i < cnt * cols_per_block; i += DR_THREADS) {
            int tt = i / cols_per_block, c = i - tt * cols_per_block;
            size_t n = (size_t)(start + t0 + tt);
            vs[i] = (c0 + c < vdim) ? v[(n * heads + head) * vdim + c0 + c] : 0.f;
        }
        if (tid < cnt) bs[tid] = beta[(size_t)(start + t0 + tid) * heads + head];
        __syncthreads();
        for (int tt = 0; tt < cnt; ++tt) {
            const float* kt = ks + tt * dim;
            const float* qt = qs + tt * dim;
            const float* gt = gs + tt * dim;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                int r = sub + i * tpc;
                if (r < dim) {
                    s[i] *= gt[r];
                    dot = fmaf(s[i], kt[r], dot);
                }
            }
            for (int o = tpc >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            float u = bs[tt] * (vs[tt * cols_per_block + tid / tpc] - dot);
            float rd = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                int r = sub + i * tpc;
                if (r < dim) {
                    s[i] = fmaf(kt[r], u, s[i]);
                    rd = fmaf(s[i], qt[r], rd);
                }
            }
            for (int o = tpc >> 1; o > 0; o >>= 1) rd += __shfl_xor_sync(0xffffffffu, rd, o);
            if (live && sub == 0) out[((size_t)(start + t0 + tt) * heads + head) * vdim + col] = rd;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            int r = sub + i * tpc;
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
    size_t smem = (size_t)2 * kv_heads * dim * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    int e = ie_launch(delta_prep_kernel, dim3(num_tokens), dim3(256), smem, s, qkvb, ld, a, conv_w, A_log, dt_bias,
                      (const float*)state, state_stride, slots, seq_of_token, cu_q, q_out, k_out, v_out, beta,
                      decay, heads, kv_heads, dim, vdim, taps, num_slots, err);
    if (e != 0 || taps < 2) return e;
    int channels = 2 * kv_heads * dim + heads * vdim;
    return ie_launch(delta_conv_tail_kernel, dim3(num_seqs), dim3(256), 0, s, qkvb, ld, state, state_stride, slots,
                     cu_q, (long long)heads * dim * vdim, channels, taps, num_slots);
}

IE_API int ie_delta_rule(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                         float* state, long long state_stride, const int* slots, const int* cu_q, float* out,
                         int num_seqs, int heads, int kv_heads, int dim, int vdim, int num_slots, void* stream) {
    if (num_seqs <= 0) return 0;
    constexpr int R = 16;
    int tpc = 1;
    while (tpc * R < dim) tpc *= 2;
    if (tpc > 32) return (int)cudaErrorInvalidValue;  // dim <= 512
    int cols = DR_THREADS / tpc;
    dim3 grid((vdim + cols - 1) / cols, heads, num_seqs);
    size_t smem = ((size_t)DR_CHUNK * (3 * dim + cols) + DR_CHUNK) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return ie_launch(delta_rule_kernel<R>, grid, dim3(DR_THREADS), smem, (cudaStream_t)stream, q, k, v, beta, decay,
                     state, state_stride, slots, cu_q, out, heads, kv_heads, dim, vdim, tpc, num_slots);
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
