// Kernels of the latent attention mixer besides the attention itself (which is the general paged
// kernel with value rows inside the key rows):
//
//  * latent_prep: from the fused input projection's 32-bit output, per token: the queries'
//    unrotated parts, the queries' rotated parts (turned, written behind the latent part of the
//    query rows the attention reads), the heads' output gates, and the cached row: the latent
//    (divided by its root mean square, times a weight) followed by the shared rotated key part.
//  * headwise_linear: out[n, h, :] = W[h] x[n, h, :] (times an optional factor per token and
//    head): the products that move the per-head key and value matrices to the query side.
//
// Rotation: entries 2i and 2i+1 of the rotated part form a pair for i < rot_dims / 2,
// (u, v) -> (u cos a - v sin a, v cos a + u sin a) with a = position * base^(-2i / rot_dims) from the
// 32-bit table [positions, 2, rot_dims / 2]; entries from rot_dims on pass unchanged.
// All arithmetic is 32-bit; results are rounded once to the output's dtype.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ positions,
                   const float* __restrict__ table, int rot_dims, int table_rows,
                   const float* __restrict__ norm_w, float eps, T* __restrict__ q_plain,
                   T* __restrict__ q_abs, float* __restrict__ gate, T* __restrict__ cache,
                   const int* __restrict__ slot_mapping, int heads, int dim, int rot_dim, int rank,
                   int total_slots, int* err) {
    __shared__ float red[4];
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x, tid = threadIdx.x;
    const float* row = proj + (size_t)n * ld;
    int hq = dim + rot_dim, krow = rank + rot_dim;
    int pos = positions[n];
    bool turn = table != nullptr && rot_dims > 0;
    if (turn && (pos < 0 || pos >= table_rows)) {
        if (tid == 0) ie_report(err, IE_ERR_POSITION, pos, n);
        turn = false;
    }
    const float* cs = turn ? table + (size_t)pos * rot_dims : nullptr;  // cos [rot_dims/2], then sin
    int half = rot_dims / 2;

    // queries: unrotated parts as they are, rotated parts behind the latent part of the query rows
    for (int i = tid; i < heads * dim; i += blockDim.x) {
        int h = i / dim, d = i - h * dim;
        ie_store(q_plain + (size_t)n * heads * dim + i, row[h * hq + d]);
    }
    for (int i = tid; i < heads * rot_dim; i += blockDim.x) {
        int h = i / rot_dim, d = i - h * rot_dim;
        const float* src = row + h * hq + dim;
        float v = src[d];
        if (turn && d < rot_dims) {
            int j = d >> 1;
            float c = cs[j], s = cs[half + j];
            v = (d & 1) ? fmaf(src[d], c, src[d - 1] * s) : fmaf(src[d], c, -src[d + 1] * s);
        }
        ie_store(q_abs + ((size_t)n * heads + h) * krow + rank + d, v);
    }
    const float* dkv = row + heads * hq;
    const float* g = dkv + krow;
    for (int h = tid; h < heads; h += blockDim.x) gate[(size_t)n * heads + h] = 1.0f / (1.0f + expf(-g[h]));

    if (slot_mapping == nullptr) return;  // a run that borrows another layer's cache writes none
    int slot = slot_mapping[n];
    if (slot < 0 || slot >= total_slots) {
        if (tid == 0) ie_report(err, IE_ERR_PAGE, slot, n);
        return;
    }
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) ss = fmaf(dkv[i], dkv[i], ss);
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)rank + eps);
    T* dst = cache + (size_t)slot * krow;
    for (int i = tid; i < rank; i += blockDim.x) ie_store(dst + i, dkv[i] * inv * norm_w[i]);
    for (int d = tid; d < rot_dim; d += blockDim.x) {
        const float* src = dkv + rank;
        float v = src[d];
        if (turn && d < rot_dims) {
            int j = d >> 1;
            float c = cs[j], s = cs[half + j];
            v = (d & 1) ? fmaf(src[d], c, src[d - 1] * s) : fmaf(src[d], c, -src[d + 1] * s);
        }
        ie_store(dst + rank + d, v);
    }
}

// out[n, h, o] = scale[n, h] * sum_k x[n, h, k] * W[h, o, k], k ascending per output.
// x rows: x + n * x_ld + h * x_hs; out rows: out + n * o_ld + h * o_hs.  Tiles of 32 tokens x 32
// outputs of one head; each of 256 threads owns a 2 x 2 patch.
constexpr int HB = 32, HK = 32;

template <typename T>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const T* __restrict__ x, long long x_ld, long long x_hs, const T* __restrict__ w,
                       T* __restrict__ out, long long o_ld, long long o_hs,
                       const float* __restrict__ scale, int N, int heads, int O, int K) {
    __shared__ float xs[HK][HB + 1];
    __shared__ float ws[HK][HB + 1];
    ie_pdl_trigger();
    ie_pdl_wait();
    int h = blockIdx.z, n0 = blockIdx.y * HB, o0 = blockIdx.x * HB;
    int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const T* wh = w + (size_t)h * O * K;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += HK) {
        for (int i = tid; i < HB * HK; i += 256) {
            int r = i / HK, k = i - r * HK;
            float xv = 0.f, wv = 0.f;
            if (k0 + k < K) {
                if (n0 + r < N) xv = ie_load(x + (size_t)(n0 + r) * x_ld + (size_t)h * x_hs + k0 + k);
                if (o0 + r < O) wv = ie_load(wh + (size_t)(o0 + r) * K + k0 + k);
            }
            xs[k][r] = xv;
            ws[k][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HK; ++k) {
            float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1], b0 = ws[k][tx * 2], b1 = ws[k][tx * 2 + 1];
            acc[0][0] = fmaf(a0, b0, acc[0][0]); acc[0][1] = fmaf(a0, b1, acc[0][1]);
            acc[1][0] = fmaf(a1, b0, acc[1][0]); acc[1][1] = fmaf(a1, b1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        int n = n0 + ty * 2 + i;
        if (n >= N) continue;
        float f = scale ? scale[(size_t)n * heads + h] : 1.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int o = o0 + tx * 2 + j;
            if (o < O) ie_store(out + (size_t)n * o_ld + (size_t)h * o_hs + o, acc[i][j] * f);
        }
    }
}
// out[n, h, :] *= scale[n, h] (bfloat16 rows of `o` entries, rows n * o_ld + h * o_hs apart)
__global__ void scale_head_rows_kernel(__nv_bfloat16* __restrict__ out, long long o_ld, long long o_hs,
                                       const float* __restrict__ scale, int heads, int o) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x;
    for (int i = threadIdx.x; i < heads * o; i += blockDim.x) {
        int h = i / o, c = i - h * o;
        __nv_bfloat16* p = out + (size_t)n * o_ld + (size_t)h * o_hs + c;
        *p = __float2bfloat16_rn(__bfloat162float(*p) * scale[(size_t)n * heads + h]);
    }
}
}  // namespace

IE_API int ie_scale_head_rows(void* out, long long o_ld, long long o_hs, const float* scale, int N, int heads, int o,
                              void* stream) {
    if (N <= 0) return 0;
    return ie_launch(scale_head_rows_kernel, dim3(N), dim3(256), 0, (cudaStream_t)stream, (__nv_bfloat16*)out, o_ld, o_hs,
                     scale, heads, o);
}

IE_API int ie_latent_prep(const float* proj, int ld, const int* positions, const float* table, int rot_dims,
                          int table_rows, const float* norm_w, float eps, void* q_plain, void* q_abs,
                          float* gate, void* cache, int dtype, const int* slot_mapping, int num_tokens,
                          int heads, int dim, int rot_dim, int rank, int total_slots, int* err, void* stream) {
    if (num_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16)
        return ie_launch(latent_prep_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, s, proj, ld, positions,
                         table, rot_dims, table_rows, norm_w, eps, (__nv_bfloat16*)q_plain, (__nv_bfloat16*)q_abs,
                         gate, (__nv_bfloat16*)cache, slot_mapping, heads, dim, rot_dim, rank, total_slots, err);
    return ie_launch(latent_prep_kernel<float>, dim3(num_tokens), dim3(128), 0, s, proj, ld, positions, table,
                     rot_dims, table_rows, norm_w, eps, (float*)q_plain, (float*)q_abs, gate, (float*)cache,
                     slot_mapping, heads, dim, rot_dim, rank, total_slots, err);
}

IE_API int ie_headwise_linear(const void* x, long long x_ld, long long x_hs, const void* w, void* out,
                              long long o_ld, long long o_hs, const float* scale, int dtype, int N, int heads,
                              int O, int K, void* stream) {
    if (N <= 0 || heads <= 0 || O <= 0) return 0;
    dim3 grid((O + HB - 1) / HB, (N + HB - 1) / HB, heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16)
        return ie_launch(headwise_linear_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x, x_ld,
                         x_hs, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_ld, o_hs, scale, N, heads, O, K);
    return ie_launch(headwise_linear_kernel<float>, grid, dim3(256), 0, s, (const float*)x, x_ld, x_hs,
                     (const float*)w, (float*)out, o_ld, o_hs, scale, N, heads, O, K);
}
