// Attention over shared latent rows on the tensor cores (bfloat16).
//
// Every query head of a token attends over the same cached rows: a key is a whole row (DK
// entries: the latent, then the rotated part), its value the row's first DV entries.  So the rows
// of the score matrix are (token, head) pairs of one request, and a block streams the request's
// rows once for all of its pairs: 16 pairs and 64-key tiles where requests bring a token or two
// (decoding), 64 pairs and 32-key tiles where they bring portions of prompts (a key tile then
// serves four times the rows).  Eight warps:
//   scores   a warp takes eight keys of the tile (and a share of the rows' 16-row tiles):
//            S = Q K^T over DK by mma.sync.m16n8k16, Q and the key tile in shared memory (key tiles
//            arrive by cp.async, two buffers);
//   softmax  a few threads per row: mask (a row sees positions up to its own), running maximum
//            and sum in 32-bit, weights rounded to bfloat16 into shared memory;
//   values   warp w owns every eighth 8-column slice of the DV output columns: O = O * alpha + P V,
//            V's fragments straight from the key tile with ldmatrix.trans.
// A context may be cut into `splits` ranges of key tiles (few requests, long contexts): the blocks of
// a range leave maximum, sum and the unnormalised output in scratch, and a second kernel adds the
// ranges in order.  Rows, sums and the order of additions depend on the request alone.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int LM_MAX_DV = 512;  // value rows of up to this many entries (64 8-column slices dealt over the warps)

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, const unsigned* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

struct LmSmem {
    __nv_bfloat16* q;   // [rows][ld]
    __nv_bfloat16* k;   // [2][keys][ld]
    float* s;           // [rows][keys + 4]
    __nv_bfloat16* p;   // [rows][keys + 8]
    float* alpha;       // [rows]
    float* m;           // [rows]
    float* l;           // [rows]
};

inline __host__ __device__ int lm_ld(int dk) { return ((dk + 15) / 16) * 16 + 8; }
inline size_t lm_smem_bytes(int dk, int rows, int keys) {
    size_t ld = lm_ld(dk);
    return (rows + 2 * keys) * ld * 2 + rows * (keys + 4) * 4 + rows * (keys + 8) * 2 + 3 * rows * 4;
}

// grid: (row tiles of a request, requests, splits).  MT 16-row tiles and KEYS keys per step, LM_WARPS warps.
template <int MT, int KEYS, int LM_WARPS>
__global__ void __launch_bounds__(LM_WARPS * 32)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                            const int* __restrict__ block_tables, int table_width, const int* __restrict__ cu_q,
                            const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ scratch, int heads, int dk, int dv, int page_size,
                            int total_pages, float scale, int splits, int* err) {
    extern __shared__ __align__(16) unsigned char raw[];
    constexpr int LM_ROWS = 16 * MT, LM_KEYS = KEYS, LM_THREADS = LM_WARPS * 32;
    constexpr int LM_MAX_NT = LM_MAX_DV / 8 / LM_WARPS;  // 8-column slices of the output per warp
    constexpr int N_TILES = KEYS / 8;            // 8-key slices of a key tile
    constexpr int WPN = LM_WARPS / N_TILES;      // warps that share a slice, each with MT / WPN row tiles
    constexpr int MPW = MT / WPN;
    constexpr int TPR = LM_THREADS / LM_ROWS;    // softmax threads per row
    constexpr int KPT = KEYS / TPR;              // ... and keys per thread
    static_assert(LM_WARPS % N_TILES == 0 && MT % WPN == 0 && MPW >= 1 && KPT % 4 == 0 && TPR <= 32, "shape");
    ie_pdl_trigger();
    ie_pdl_wait();
    // (the blocks of a request's last rows see the most keys: they start first)
    int seq = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.z;
    int q0 = cu_q[seq], q_len = cu_q[seq + 1] - q0;
    int rows_total = q_len * heads;
    int row0 = tile * LM_ROWS;
    if (row0 >= rows_total) return;
    int ctx_len = ctx_lens[seq];
    int start = ctx_len - q_len;  // position of the request's first token of this step
    int rows_here = min(LM_ROWS, rows_total - row0);
    int last_pos = start + (row0 + rows_here - 1) / heads;  // the last position any row of the block sees
    int tiles_all = last_pos / LM_KEYS + 1;
    int per = (tiles_all + splits - 1) / splits;
    int t_begin = split * per, t_end = min(tiles_all, t_begin + per);

    int ld = lm_ld(dk);
    LmSmem sm;
    sm.q = reinterpret_cast<__nv_bfloat16*>(raw);
    sm.k = sm.q + LM_ROWS * ld;
    sm.s = reinterpret_cast<float*>(sm.k + 2 * LM_KEYS * ld);
    sm.p = reinterpret_cast<__nv_bfloat16*>(sm.s + LM_ROWS * (LM_KEYS + 4));
    sm.alpha = reinterpret_cast<float*>(sm.p + LM_ROWS * (LM_KEYS + 8));
    sm.m = sm.alpha + LM_ROWS;
    sm.l = sm.m + LM_ROWS;

    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int* table = block_tables + (size_t)seq * table_width;
    int chunks = dk / 8;  // 16-byte pieces of a row
    int page_shift = 31 - __clz(page_size);  // (pages hold a power of two of tokens)

    // columns beyond dk (up to the next multiple of 16) must read as zero in both operands
    int dkp = ld - 8;
    if (dkp > dk) {
        for (int i = tid; i < (LM_ROWS + 2 * LM_KEYS) * (dkp - dk); i += LM_THREADS) {
            int r = i / (dkp - dk), c = dk + i % (dkp - dk);
            sm.q[r * ld + c] = __float2bfloat16_rn(0.f);  // (q and k are one array of rows)
        }
    }
    auto load_keys = [&](int t, int buf) {
        __nv_bfloat16* dst = sm.k + (size_t)buf * LM_KEYS * ld;
        for (int key = warp; key < LM_KEYS; key += LM_WARPS) {  // a warp takes whole keys, its lanes their pieces
            int pos = t * LM_KEYS + key;
            const __nv_bfloat16* src = cache;
            int bytes = 0;
            if (pos <= last_pos) {
                int page = table[pos >> page_shift];
                if (page < 0 || page >= total_pages) ie_report(err, page < 0 ? IE_ERR_TABLE : IE_ERR_PAGE, page, seq);
                else {
                    src = cache + ((size_t)page * page_size + (pos & (page_size - 1))) * dk;
                    bytes = 16;
                }
            }
            __nv_bfloat16* drow = dst + key * ld;
            for (int c = lane; c < chunks; c += 32) cp_async16(drow + c * 8, bytes ? src + c * 8 : cache, bytes);
        }
        cp_async_commit();
    };
    if (t_begin < t_end) load_keys(t_begin, 0);
    // queries: row r of the block is (token (row0 + r) / heads, head (row0 + r) % heads)
    for (int i = tid; i < LM_ROWS * chunks; i += LM_THREADS) {
        int r = i / chunks, c = i - r * chunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows_here) {
            int rr = row0 + r;
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(q0 + rr / heads) * heads + rr % heads) * dk + c * 8);
        }
        *reinterpret_cast<uint4*>(sm.q + r * ld + c * 8) = v;
    }
    if (tid < LM_ROWS) { sm.m[tid] = -INFINITY; sm.l[tid] = 0.f; }

    float acc[MT][LM_MAX_NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < LM_MAX_NT; ++i) acc[mt][i][0] = acc[mt][i][1] = acc[mt][i][2] = acc[mt][i][3] = 0.f;
    int n_tiles = (dv + 7) / 8;  // 8-column slices of the output; warp w owns slices w, w + 8, ...

    for (int t = t_begin; t < t_end; ++t) {
        int buf = (t - t_begin) & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (t + 1 < t_end) load_keys(t + 1, buf ^ 1);
        const __nv_bfloat16* ks = sm.k + (size_t)buf * LM_KEYS * ld;
        // scores: this warp's eight keys against its row tiles
        {
            int ns = warp % N_TILES, m_first = (warp / N_TILES) * MPW;
            float c[MPW][4];
#pragma unroll
            for (int i = 0; i < MPW; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
            // fragments by ldmatrix: A (16 x 16 of Q) one x4; B (8 keys x 32 of k) one x4 for two steps
            unsigned qa = (unsigned)__cvta_generic_to_shared(sm.q + (m_first * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
            unsigned kb = (unsigned)__cvta_generic_to_shared(ks + (ns * 8 + (lane & 7)) * ld + (lane >> 3) * 8);
            int kk = 0;
            for (; kk + 32 <= dkp; kk += 32) {
                unsigned b[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(kb + kk * 2));
                // (all fragments of the 32 columns first, then the products: a load's latency is paid
                // once per 32 columns, not once per product)
                unsigned a[MPW][2][4];
#pragma unroll
                for (int i = 0; i < MPW; ++i)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(a[i][h][0]), "=r"(a[i][h][1]), "=r"(a[i][h][2]), "=r"(a[i][h][3])
                                     : "r"(qa + (i * 16 * ld + kk + h * 16) * 2));
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < MPW; ++i) mma_bf16(c[i], a[i][h], b + 2 * h);
            }
            if (kk < dkp) {  // a last step of 16
                unsigned b[2];
                unsigned kb2 = (unsigned)__cvta_generic_to_shared(ks + (ns * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                             : "=r"(b[0]), "=r"(b[1]) : "r"(kb2 + kk * 2));
#pragma unroll
                for (int i = 0; i < MPW; ++i) {
                    unsigned a[4];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(qa + (i * 16 * ld + kk) * 2));
                    mma_bf16(c[i], a, b);
                }
            }
#pragma unroll
            for (int i = 0; i < MPW; ++i) {
                float* s0 = sm.s + ((m_first + i) * 16 + g) * (LM_KEYS + 4) + ns * 8 + 2 * t4;
                s0[0] = c[i][0] * scale; s0[1] = c[i][1] * scale;
                s0[8 * (LM_KEYS + 4)] = c[i][2] * scale; s0[8 * (LM_KEYS + 4) + 1] = c[i][3] * scale;
            }
        }
        __syncthreads();
        // softmax: TPR threads per row, KPT keys each
        {
            int r = tid / TPR, j = tid % TPR;
            int rr = row0 + r;
            int pos_r = r < rows_here ? start + rr / heads : -1;
            float v[KPT], mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                int kp = t * LM_KEYS + j * KPT + i;
                v[i] = kp <= pos_r ? sm.s[r * (LM_KEYS + 4) + j * KPT + i] : -INFINITY;
                mx = fmaxf(mx, v[i]);
            }
#pragma unroll
            for (int o = TPR / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float m_old = sm.m[r];
            float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            __align__(8) __nv_bfloat16 pb[KPT];
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                float pv = (v[i] == -INFINITY) ? 0.f : expf(v[i] - m_new);
                pb[i] = __float2bfloat16_rn(pv);
                sum += pv;
            }
#pragma unroll
            for (int o = TPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
            for (int i = 0; i < KPT; i += 4)
                *reinterpret_cast<uint2*>(sm.p + r * (LM_KEYS + 8) + j * KPT + i) = *reinterpret_cast<uint2*>(pb + i);
            if (j == 0) {
                float a = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
                if (m_new == -INFINITY) a = 1.f;
                sm.alpha[r] = a;
                sm.m[r] = m_new;
                sm.l[r] = sm.l[r] * a + sum;
            }
        }
        __syncthreads();
        // values
        {
            unsigned pa[MT][LM_KEYS / 16][4];
            float a0[MT], a1[MT];
            bool moved = false;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                a0[mt] = sm.alpha[mt * 16 + g];
                a1[mt] = sm.alpha[mt * 16 + g + 8];
                moved = moved || a0[mt] != 1.f || a1[mt] != 1.f;
                unsigned pr = (unsigned)__cvta_generic_to_shared(sm.p + (mt * 16 + (lane & 15)) * (LM_KEYS + 8) + (lane >> 4) * 8);
#pragma unroll
                for (int kk = 0; kk < LM_KEYS / 16; ++kk)
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(pa[mt][kk][0]), "=r"(pa[mt][kk][1]), "=r"(pa[mt][kk][2]), "=r"(pa[mt][kk][3])
                                 : "r"(pr + kk * 32));
            }
            moved = __any_sync(0xffffffffu, moved);  // (mostly false once the rows' maxima have settled)
#pragma unroll
            for (int i = 0; i < LM_MAX_NT; ++i) {
                int nt = warp + i * LM_WARPS;
                if (nt >= n_tiles) break;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (moved) { acc[mt][i][0] *= a0[mt]; acc[mt][i][1] *= a0[mt]; acc[mt][i][2] *= a1[mt]; acc[mt][i][3] *= a1[mt]; }
                }
                unsigned b[LM_KEYS / 16][2];
#pragma unroll
                for (int kk = 0; kk < LM_KEYS / 16; ++kk) {
                    unsigned addr = (unsigned)__cvta_generic_to_shared(ks + (kk * 16 + (lane & 15)) * ld + nt * 8);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                                 : "=r"(b[kk][0]), "=r"(b[kk][1]) : "r"(addr));
                }
#pragma unroll
                for (int kk = 0; kk < LM_KEYS / 16; ++kk)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) mma_bf16(acc[mt][i], pa[mt][kk], b[kk]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    // write: normalised if the block saw the whole context, else the parts for the second kernel
#pragma unroll
    for (int i = 0; i < LM_MAX_NT; ++i) {
        int nt = warp + i * LM_WARPS;
        if (nt >= n_tiles) break;
#pragma unroll
        for (int mh = 0; mh < 2 * MT; ++mh) {
            int mt = mh >> 1, half = mh & 1;
            int r = mt * 16 + g + half * 8;
            if (r >= rows_here) continue;
            int rr = row0 + r;
            int col = nt * 8 + 2 * t4;
            float v0 = acc[mt][i][half * 2], v1 = acc[mt][i][half * 2 + 1];
            if (splits == 1) {
                float inv = sm.l[r] > 0.f ? 1.0f / sm.l[r] : 0.f;
                __nv_bfloat16* dst = out + ((size_t)(q0 + rr / heads) * heads + rr % heads) * dv + col;
                if (col < dv) dst[0] = __float2bfloat16_rn(v0 * inv);
                if (col + 1 < dv) dst[1] = __float2bfloat16_rn(v1 * inv);
            } else {
                float* dst = scratch + (((size_t)(q0 * heads + rr)) * splits + split) * (dv + 2) + 2 + col;
                if (col < dv) dst[0] = v0;
                if (col + 1 < dv) dst[1] = v1;
            }
        }
    }
    if (splits > 1 && tid < rows_here) {
        float* dst = scratch + (((size_t)(q0 * heads + row0 + tid)) * splits + split) * (dv + 2);
        dst[0] = sm.m[tid];
        dst[1] = sm.l[tid];
    }
}

// One block per (token, head) row: the ranges' parts added in order.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out, int dv, int splits) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t row = blockIdx.x;
    const float* base = scratch + row * splits * (dv + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, base[(size_t)s * (dv + 2)]);
    float l = 0.f;
    for (int s = 0; s < splits; ++s) {
        float ms = base[(size_t)s * (dv + 2)];
        if (ms != -INFINITY) l += base[(size_t)s * (dv + 2) + 1] * expf(ms - m);
    }
    float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s) {
            float ms = base[(size_t)s * (dv + 2)];
            if (ms != -INFINITY) o = fmaf(base[(size_t)s * (dv + 2) + 2 + c], expf(ms - m), o);
        }
        out[row * dv + c] = __float2bfloat16_rn(o * inv);
    }
}

IePerDevice g_lm_smem, g_lm_smem64;
}  // namespace

// Whether the tensor-core kernel takes these sizes (else the general kernel runs).
IE_API int ie_latent_attention_mma_ok(int dk, int dv) {
    return dk % 8 == 0 && dv % 8 == 0 && dv <= LM_MAX_DV && dv <= dk &&
           lm_smem_bytes(dk, 16, 64) <= 220 * 1024 && lm_smem_bytes(dk, 64, 32) <= 220 * 1024;
}

// Rows (token, head pairs) a block takes: 64 when the step's longest request brings at least that
// many (portions of prompts), else 16.
IE_API int ie_latent_attention_rows(int longest_rows) { return longest_rows >= 64 ? 64 : 16; }

// scratch floats for `splits` > 1: tokens * heads * splits * (dv + 2)
IE_API int ie_latent_attention_mma(const void* q, const void* cache, const int* block_tables, int table_width,
                                   const int* cu_q, const int* ctx_lens, void* out, float* scratch, int num_tokens,
                                   int num_seqs, int max_tiles, int rows, int heads, int dk, int dv, int page_size,
                                   int total_pages, float scale, int splits, int* err, void* stream) {
    if (num_seqs <= 0 || max_tiles <= 0) return 0;
    if (!ie_latent_attention_mma_ok(dk, dv) || splits < 1 || (splits > 1 && scratch == nullptr)) return (int)cudaErrorInvalidValue;
    if (rows != 16 && rows != 64) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
#define IE_LM_ARGS (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, table_width, cu_q, ctx_lens, \
                   (__nv_bfloat16*)out, scratch, heads, dk, dv, page_size, total_pages, scale, splits, err
    if (rows == 64) {
        // (sixteen warps instead of eight take as long: 636 against 633 us on 2,048 tokens of 16 heads)
        cudaError_t e = ie_allow_smem(g_lm_smem64, latent_attention_mma_kernel<4, 32, 8>, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
        rc = ie_launch(latent_attention_mma_kernel<4, 32, 8>, dim3(max_tiles, num_seqs, splits), dim3(8 * 32),
                       lm_smem_bytes(dk, 64, 32), s, IE_LM_ARGS);
    } else {
        cudaError_t e = ie_allow_smem(g_lm_smem, latent_attention_mma_kernel<1, 64, 8>, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
        rc = ie_launch(latent_attention_mma_kernel<1, 64, 8>, dim3(max_tiles, num_seqs, splits), dim3(8 * 32),
                       lm_smem_bytes(dk, 16, 64), s, IE_LM_ARGS);
    }
#undef IE_LM_ARGS
    if (rc != 0 || splits == 1) return rc;
    return ie_launch(latent_attention_merge_kernel, dim3(num_tokens * heads), dim3(128), 0, s, (const float*)scratch,
                     (__nv_bfloat16*)out, dv, splits);
}
