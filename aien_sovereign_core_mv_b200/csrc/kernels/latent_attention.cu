// Attention over a cached latent: per token the cache keeps one row [c | k_rot] of kv_rank + rot_dim
// numbers, shared by all heads.  c is the normed latent from which a head's unrotated key W_uk,h c and
// value W_uv,h c would be made, k_rot one rotated key part.  The kernels here work on the latent
// itself: with q_lat,h = W_uk,h^T q_h (made by a product per head) the score of head h against key j is
//     (q_lat,h . c_j + q_rot,h . k_rot,j) * scale
// and the weighted sum of values is W_uv,h (sum_j p_j c_j), so one row per key serves every head as key
// and as value, and nothing per head is ever cached or rebuilt.  Rotation, scores, softmax (with an
// optional sink per head) and the weighted sum are float32 in both engine precisions.
#include "common.cuh"
#include <math.h>

namespace aien {

// ---------------------------------------------------------------- after the down projections
// d [T, ld] float32 holds, per token, the query latent (q_rank numbers at column 0) and, when the layer
// writes a cache, the key/value latent (kv_rank numbers at kv_off) followed by rot_dim numbers of the
// shared key part.  cq = RMS norm of the query latent with weight wq; the cache row of the token
// (slot_map[t], -1: none) gets the RMS norm of the key/value latent with weight wkv, then the key part
// with its first rot_dims numbers rotated in neighbouring pairs (2i, 2i+1) by the token's angle.
template <typename TD, typename TO, typename TKV>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const TD* __restrict__ d, long ld, int q_rank, const void* __restrict__ wq, int wdt, float eps,
                      TO* __restrict__ cq, long ldq, int kv_off, int kv_rank, int rot_dim, int rot_dims,
                      const void* __restrict__ wkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      const int* __restrict__ slot_map, TKV* __restrict__ cache) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    const TD* row = d + t * ld;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_f(row[i]);
            ss += v * v;
        }
        const float sc = 1.0f / sqrtf(block_sum(ss, red) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq[t * ldq + i] = from_f<TO>(to_f(row[i]) * sc * load_dyn(wq, wdt, i));
    }
    if (cache == nullptr) return;
    const int slot = slot_map[t];
    if (slot < 0) return;                         // uniform over the block
    TKV* dst = cache + (size_t)slot * (kv_rank + rot_dim);
    float ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const float v = to_f(row[kv_off + i]);
        ss += v * v;
    }
    const float sc = 1.0f / sqrtf(block_sum(ss, red) / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
        dst[i] = from_f<TKV>(to_f(row[kv_off + i]) * sc * load_dyn(wkv, wdt, i));
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        float v = to_f(row[kv_off + kv_rank + i]);
        if (i < rot_dims) {
            const int p = i >> 1;
            const float c = cos_t[t * half + p], s = sin_t[t * half + p];
            const float other = to_f(row[kv_off + kv_rank + (i ^ 1)]);
            v = (i & 1) ? v * c + other * s : v * c - other * s;
        }
        dst[kv_rank + i] = from_f<TKV>(v);
    }
}

// The rotated part of every query head, moved behind the head's latent query:
// out[t, h, 0:rot_dim] = rotate(q[t, h, 0:rot_dim]) (first rot_dims numbers in pairs), the rotation in float32.
template <typename TQ, typename TO>
__global__ void rotate_pairs_rows_kernel(const TQ* __restrict__ q, long ldq, long q_head, TO* __restrict__ out, long ldo,
                                         long o_head, int H, int rot_dim, int rot_dims, const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t) {
    const size_t t = blockIdx.x;
    const int half = rot_dims >> 1;
    for (int idx = threadIdx.x; idx < H * rot_dim; idx += blockDim.x) {
        const int h = idx / rot_dim, i = idx % rot_dim;
        const TQ* src = q + t * ldq + (size_t)h * q_head;
        float v = to_f(src[i]);
        if (i < rot_dims) {
            const int p = i >> 1;
            const float c = cos_t[t * half + p], s = sin_t[t * half + p];
            const float other = to_f(src[i ^ 1]);
            v = (i & 1) ? v * c + other * s : v * c - other * s;
        }
        out[t * ldo + (size_t)h * o_head + i] = from_f<TO>(v);
    }
}

// ---------------------------------------------------------------- one product per head
// C[t, h, n] = sum_k A[t, h, k] * W[h, n, k]: every head multiplies its own slice of the rows by its own
// matrix (stored [out, in] like every weight).  Float32 sums on the CUDA cores, k in order, so a row's
// result depends on that row alone.  a_head / c_head: distance between heads inside a row.
constexpr int HP_BM = 64, HP_BN = 64, HP_BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
head_project_kernel(const TA* __restrict__ A, long lda, long a_head, const TW* __restrict__ W, long ldw, long w_head,
                    TC* __restrict__ C, long ldc, long c_head, int M, int N, int K) {
    __shared__ float As[HP_BK][HP_BM + 4];
    __shared__ float Ws[HP_BK][HP_BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * HP_BM, n0 = blockIdx.x * HP_BN, h = blockIdx.z;
    A += (size_t)h * a_head;
    W += (size_t)h * w_head;
    C += (size_t)h * c_head;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HP_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, c = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_f(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HP_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_f<TC>(acc[i][j]);
        }
    }
}

// ---------------------------------------------------------------- attention over the latent rows
// One CTA per (query token, block of LT_ROWS heads); LT_WARPS warps, each with LT_RPW heads.  Keys are
// visited in position order in tiles of 32: the tile's rows go to shared memory as float32 once and
// serve every head of the block, first as keys (a lane per key, the head's query broadcast), then as
// values (a lane per channel, CPL channels a lane: kv_rank <= 32 * CPL).  Online softmax per head; the
// sink joins the denominator at the end.  A token at position p sees the keys at max(0, p - window + 1)
// .. p of its request (window 0: all), read through the request's block table, so the result depends
// on the token's position and the cache alone.
constexpr int LT_WARPS = 4, LT_RPW = 4, LT_ROWS = LT_WARPS * LT_RPW, LT_KEYS = 32;

template <typename TKV, typename TO, int CPL>
__global__ void __launch_bounds__(LT_WARPS * 32)
latent_attention_kernel(const float* __restrict__ q, long ldq, const TKV* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_of_token,
                        const int* __restrict__ positions, const int* __restrict__ token_list, TO* __restrict__ out, long ldo,
                        int H, int r, int rd, int page_size, int window, float scale, const float* __restrict__ sinks) {
    extern __shared__ float sm[];
    const int D = r + rd, Dp = D + 1;
    float* Qs = sm;                          // [LT_ROWS][D]
    float* Ks = Qs + LT_ROWS * D;            // [LT_KEYS][D+1]
    float* Ps = Ks + LT_KEYS * Dp;           // [LT_ROWS][LT_KEYS]
    __shared__ int slots[LT_KEYS];
    const int t = token_list ? token_list[blockIdx.y] : blockIdx.y;
    const int h0 = blockIdx.x * LT_ROWS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    for (int idx = tid; idx < LT_ROWS * D; idx += LT_WARPS * 32) {
        const int row = idx / D, d = idx % D;
        Qs[idx] = (h0 + row < H) ? q[(size_t)t * ldq + (size_t)(h0 + row) * D + d] : 0.f;
    }
    float m[LT_RPW], l[LT_RPW], acc[LT_RPW][CPL];
#pragma unroll
    for (int i = 0; i < LT_RPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int u = 0; u < CPL; ++u) acc[i][u] = 0.f;
    }
    for (int base = start; base <= pos; base += LT_KEYS) {
        __syncthreads();                     // the tile before is used up (and Qs is written, the first time)
        if (tid < LT_KEYS) {
            const int j = base + tid;
            int slot = -1;
            if (j <= pos) {
                const int page = bt[j / page_size];
                if (page >= 0) slot = page * page_size + (j % page_size);
            }
            slots[tid] = slot;
        }
        __syncthreads();
        for (int jj = warp; jj < LT_KEYS; jj += LT_WARPS) {
            const int slot = slots[jj];
            float* dst = Ks + jj * Dp;
            if (slot >= 0) {
                const TKV* src = cache + (size_t)slot * D;
                for (int d = lane; d < D; d += 32) dst[d] = to_f(src[d]);
            } else {
                for (int d = lane; d < D; d += 32) dst[d] = 0.f;
            }
        }
        __syncthreads();
        // scores: lane = key
        float sc[LT_RPW];
#pragma unroll
        for (int i = 0; i < LT_RPW; ++i) sc[i] = 0.f;
        {
            const float* kr = Ks + lane * Dp;
            const float* q0 = Qs + (warp * LT_RPW) * D;
            for (int d = 0; d < D; ++d) {
                const float kv = kr[d];
#pragma unroll
                for (int i = 0; i < LT_RPW; ++i) sc[i] = fmaf(q0[i * D + d], kv, sc[i]);
            }
        }
        const bool visible = slots[lane] >= 0;
#pragma unroll
        for (int i = 0; i < LT_RPW; ++i) {
            const float s = visible ? sc[i] * scale : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            float p = 0.f, corr = 1.f;
            if (m_new != -INFINITY) {
                p = visible ? expf(s - m_new) : 0.f;
                corr = (m[i] == -INFINITY) ? 0.f : expf(m[i] - m_new);
            }
            l[i] = l[i] * corr + warp_sum(p);
#pragma unroll
            for (int u = 0; u < CPL; ++u) acc[i][u] *= corr;
            m[i] = m_new;
            Ps[(warp * LT_RPW + i) * LT_KEYS + lane] = p;
        }
        __syncwarp();
        // weighted sum of the latent rows: lane = channel
        const int n = min(LT_KEYS, pos - base + 1);
        for (int jj = 0; jj < n; ++jj) {
            float pv[LT_RPW];
#pragma unroll
            for (int i = 0; i < LT_RPW; ++i) pv[i] = Ps[(warp * LT_RPW + i) * LT_KEYS + jj];
            const float* vr = Ks + jj * Dp;
#pragma unroll
            for (int u = 0; u < CPL; ++u) {
                const int c = lane + 32 * u;
                const float v = c < r ? vr[c] : 0.f;
#pragma unroll
                for (int i = 0; i < LT_RPW; ++i) acc[i][u] = fmaf(pv[i], v, acc[i][u]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < LT_RPW; ++i) {
        const int h = h0 + warp * LT_RPW + i;
        if (h >= H) continue;
        float li = l[i], corr = 1.f;
        if (sinks != nullptr) {                           // the sink counts once, unscaled, with no value
            const float sk = sinks[h];
            const float m_new = fmaxf(m[i], sk);
            corr = (m[i] == -INFINITY) ? 0.f : expf(m[i] - m_new);
            li = li * corr + expf(sk - m_new);
        }
        const float inv = li > 0.f ? corr / li : 0.f;
#pragma unroll
        for (int u = 0; u < CPL; ++u) {
            const int c = lane + 32 * u;
            if (c < r) out[(size_t)t * ldo + (size_t)h * r + c] = from_f<TO>(acc[i][u] * inv);
        }
    }
}

template <typename TKV, typename TO, int CPL>
static int launch_latent_attention(dim3 grid, size_t smem, cudaStream_t stream, const float* q, long ldq, const TKV* cache,
                                   const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                                   const int* token_list, TO* out, long ldo, int H, int r, int rd, int page_size, int window,
                                   float scale, const float* sinks) {
    auto kern = latent_attention_kernel<TKV, TO, CPL>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<grid, LT_WARPS * 32, smem, stream>>>(q, ldq, cache, block_table, max_blocks, seq_of_token, positions, token_list, out, ldo,
                                                H, r, rd, page_size, window, scale, sinks);
    return 0;
}

template <typename TKV, typename TO>
static int dispatch_latent_attention(int cpl, dim3 grid, size_t smem, cudaStream_t stream, const float* q, long ldq, const TKV* cache,
                                     const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                                     const int* token_list, TO* out, long ldo, int H, int r, int rd, int page_size, int window,
                                     float scale, const float* sinks) {
#define LT_CASE(C)                                                                                                             \
    if (cpl <= C)                                                                                                              \
        return launch_latent_attention<TKV, TO, C>(grid, smem, stream, q, ldq, cache, block_table, max_blocks, seq_of_token,     \
                                                   positions, token_list, out, ldo, H, r, rd, page_size, window, scale, sinks)
    LT_CASE(1);
    LT_CASE(2);
    LT_CASE(4);
    LT_CASE(8);
    LT_CASE(16);
    LT_CASE(32);
#undef LT_CASE
    return AIEN_E_SHAPE;
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_latent_prepare(const void* d, int d_dt, long ld, int q_rank, const void* wq, const void* wkv, int w_dt, float eps,
                                 void* cq, int cq_dt, long ldq, int kv_off, int kv_rank, int rot_dim, int rot_dims,
                                 const float* cos_t, const float* sin_t, const int* slot_map, void* cache, int kv_dt,
                                 int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (q_rank < 0 || kv_rank < 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1)) return AIEN_E_SHAPE;
    if (cache != nullptr && (kv_rank <= 0 || slot_map == nullptr || (rot_dims > 0 && (cos_t == nullptr || sin_t == nullptr)))) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(d_dt, TD, AIEN_DISPATCH_DTYPE(cq_dt, TO, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (latent_prepare_kernel<TD, TO, TKV><<<T, 256, 0, stream>>>((const TD*)d, ld, q_rank, wq, w_dt, eps, (TO*)cq, ldq, kv_off, kv_rank,
                                                                  rot_dim, rot_dims, wkv, cos_t, sin_t, slot_map, (TKV*)cache)))));
    return launch_status();
}

AIEN_API int aien_rotate_pairs_rows(const void* q, int q_dt, long ldq, long q_head, void* out, int o_dt, long ldo, long o_head, int T, int H,
                                    int rot_dim, int rot_dims, const float* cos_t, const float* sin_t, cudaStream_t stream) {
    if (T <= 0 || H <= 0 || rot_dim <= 0) return 0;
    if (rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || (rot_dims > 0 && (cos_t == nullptr || sin_t == nullptr))) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(q_dt, TQ, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (rotate_pairs_rows_kernel<TQ, TO><<<T, 128, 0, stream>>>((const TQ*)q, ldq, q_head, (TO*)out, ldo, o_head, H, rot_dim, rot_dims, cos_t, sin_t))));
    return launch_status();
}

AIEN_API int aien_head_project(const void* A, int a_dt, long lda, long a_head, const void* W, int w_dt, long ldw, long w_head,
                               void* C, int c_dt, long ldc, long c_head, int M, int N, int K, int heads, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return 0;
    if (K <= 0 || heads > 65535) return AIEN_E_SHAPE;
    dim3 grid((N + HP_BN - 1) / HP_BN, (M + HP_BM - 1) / HP_BM, heads);
    if (grid.y > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(a_dt, TA, AIEN_DISPATCH_DTYPE(w_dt, TW, AIEN_DISPATCH_DTYPE(c_dt, TC,
        (head_project_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, lda, a_head, (const TW*)W, ldw, w_head, (TC*)C, ldc,
                                                                  c_head, M, N, K)))));
    return launch_status();
}

// q float32 [T, ldq]: per head kv_rank + rot_dim numbers (the latent query, then the rotated part).  cache [slots, kv_rank + rot_dim].
// out [T, ldo]: per head kv_rank numbers (the weighted sum of latents).  token_list (or null) names the T tokens served.
AIEN_API int aien_latent_attention(const float* q, long ldq, const void* cache, int kv_dt, const int* block_table, int max_blocks,
                                   const int* seq_of_token, const int* positions, const int* token_list, void* out, int o_dt, long ldo,
                                   int T, int H, int kv_rank, int rot_dim, int page_size, int window, float scale,
                                   const float* sinks, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || kv_rank <= 0 || rot_dim < 0 || page_size <= 0 || window < 0 || T > 65535) return AIEN_E_SHAPE;
    const int D = kv_rank + rot_dim;
    const size_t smem = (size_t)(LT_ROWS * D + LT_KEYS * (D + 1) + LT_ROWS * LT_KEYS) * sizeof(float);
    if (smem > 220 * 1024) return AIEN_E_SHAPE;
    const int cpl = (kv_rank + 31) / 32;
    dim3 grid((H + LT_ROWS - 1) / LT_ROWS, T);
    int rc = 0;
    AIEN_DISPATCH_DTYPE(kv_dt, TKV, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (rc = dispatch_latent_attention<TKV, TO>(cpl, grid, smem, stream, q, ldq, (const TKV*)cache, block_table, max_blocks, seq_of_token,
                                                 positions, token_list, (TO*)out, ldo, H, kv_rank, rot_dim, page_size, window, scale, sinks))));
    if (rc != 0) return rc;
    return launch_status();
}
