// Recurrent mixers whose state has a fixed size per request: linear attention with a per-head
// decay, and a gated recurrence over channels.  The state is float32 and lives in a state slot
// of the cache ([slots, ...]); everything that enters a recurrence (decay powers, gates,
// candidates, the state itself, the products with it) is float32 in both engine precisions.
//
// The rules of a state slot, all of them on the device: the portion of request s of the step is
// the tokens q_start[s] .. q_start[s+1]; its slot is slot_map[s]; a portion whose first token has
// position 0 starts from a zero state whatever the slot held.  A launch depends on the number of
// requests and on the sizes only, so a step can be captured or recorded.
#include "common.cuh"
#include <math.h>

namespace aien {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
// lambda^e for an integer e >= 0 from log2(lambda); e = 0 gives 1 also for lambda = 0
__device__ __forceinline__ float decay_pow(float l2, int e) { return e == 0 ? 1.0f : exp2f((float)e * l2); }

// ---------------------------------------------------------------- linear attention with decay
//   S_t = lambda_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t         (S: [dim, vdim] per head)
// with q, k, v = silu of their projections.  One CTA owns (request, head, a slice of LA_VS value
// columns): columns of the state are independent of one another.  The portion is walked in
// chunks of LA_C tokens; inside a chunk
//   A[i][j] = (q_i . k_j) lambda^(i-j), j <= i
//   o_i     = sum_j A[i][j] v_j + lambda^(i+1) S^T q_i
//   S       = lambda^n S + sum_j lambda^(n-1-j) k_j v_j^T
// which equals the token-by-token recurrence up to rounding; a chunk of one token is the
// recurrence itself.  Only powers with non-negative exponents are formed.
constexpr int LA_C = 32, LA_VS = 32, LA_THREADS = 256;

template <typename TP>
__global__ void __launch_bounds__(LA_THREADS)
decay_linear_attention_kernel(const TP* __restrict__ proj, long ld, int q_off, int k_off, int v_off,
                              const float* __restrict__ decay, float* __restrict__ state,
                              const int* __restrict__ slot_map, const int* __restrict__ q_start,
                              const int* __restrict__ positions, float* __restrict__ out, long ldo,
                              int H, int dim, int vd) {
    extern __shared__ float sm[];
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * LA_VS;
    const int nv = min(LA_VS, vd - v0);
    const int tid = threadIdx.x;
    const int dp = dim + 1;
    float* Qs = sm;                         // [LA_C][dim+1]
    float* Ks = Qs + LA_C * dp;             // [LA_C][dim+1]
    float* Vs = Ks + LA_C * dp;             // [LA_C][LA_VS]
    float* As = Vs + LA_C * LA_VS;          // [LA_C][LA_C+1]
    float* Ss = As + LA_C * (LA_C + 1);     // [dim][LA_VS]
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 <= t0) return;
    const int slot = slot_map[s];
    float* st = state + (((size_t)slot * H + h) * dim) * vd;
    const bool fresh = positions[t0] == 0;
    for (int idx = tid; idx < dim * LA_VS; idx += LA_THREADS) {
        const int d = idx / LA_VS, v = idx % LA_VS;
        Ss[idx] = (!fresh && v < nv) ? st[(size_t)d * vd + v0 + v] : 0.f;
    }
    const float lam = decay[h];
    const float l2 = log2f(lam);
    for (int c0 = t0; c0 < t1; c0 += LA_C) {
        const int n = min(LA_C, t1 - c0);
        __syncthreads();
        for (int idx = tid; idx < n * dim; idx += LA_THREADS) {
            const int i = idx / dim, d = idx % dim;
            const TP* row = proj + (size_t)(c0 + i) * ld + (size_t)h * dim + d;
            Qs[i * dp + d] = silu_f(to_f(row[q_off]));
            Ks[i * dp + d] = silu_f(to_f(row[k_off]));
        }
        for (int idx = tid; idx < n * LA_VS; idx += LA_THREADS) {
            const int i = idx / LA_VS, v = idx % LA_VS;
            Vs[idx] = v < nv ? silu_f(to_f(proj[(size_t)(c0 + i) * ld + v_off + (size_t)h * vd + v0 + v])) : 0.f;
        }
        __syncthreads();
        // scores inside the chunk
        for (int idx = tid; idx < n * LA_C; idx += LA_THREADS) {
            const int i = idx / LA_C, j = idx % LA_C;
            float a = 0.f;
            if (j <= i) {
                const float* qi = Qs + i * dp;
                const float* kj = Ks + j * dp;
                for (int d = 0; d < dim; ++d) a = fmaf(qi[d], kj[d], a);
                a *= decay_pow(l2, i - j);
            }
            As[i * (LA_C + 1) + j] = a;
        }
        __syncthreads();
        // outputs of the chunk: what the chunk's own tokens give, plus the state before the chunk
        for (int idx = tid; idx < n * LA_VS; idx += LA_THREADS) {
            const int i = idx / LA_VS, v = idx % LA_VS;
            if (v >= nv) continue;
            float intra = 0.f;
            for (int j = 0; j <= i; ++j) intra = fmaf(As[i * (LA_C + 1) + j], Vs[j * LA_VS + v], intra);
            float inter = 0.f;
            const float* qi = Qs + i * dp;
            for (int d = 0; d < dim; ++d) inter = fmaf(qi[d], Ss[d * LA_VS + v], inter);
            out[(size_t)(c0 + i) * ldo + (size_t)h * vd + v0 + v] = intra + decay_pow(l2, i + 1) * inter;
        }
        __syncthreads();
        // the state after the chunk
        const float ln = decay_pow(l2, n);
        for (int idx = tid; idx < dim * LA_VS; idx += LA_THREADS) {
            const int d = idx / LA_VS, v = idx % LA_VS;
            float acc = 0.f;
            for (int j = 0; j < n; ++j) acc = fmaf(decay_pow(l2, n - 1 - j) * Ks[j * dp + d], Vs[j * LA_VS + v], acc);
            Ss[idx] = fmaf(ln, Ss[idx], acc);
        }
    }
    __syncthreads();
    for (int idx = tid; idx < dim * LA_VS; idx += LA_THREADS) {
        const int d = idx / LA_VS, v = idx % LA_VS;
        if (v < nv) st[(size_t)d * vd + v0 + v] = Ss[idx];
    }
}

// The recurrence itself for requests that bring one token each: the state streams through once.  One CTA per (request,
// head, 32 value columns); thread (v, g) walks the rows d = g, g + 8, ... of its column: S[d][v] = lambda S[d][v] + k[d] v[v],
// o[v] += S[d][v] q[d]; the eight row groups of a column are added through shared memory in order.
template <typename TP>
__global__ void __launch_bounds__(256)
decay_linear_attention_token_kernel(const TP* __restrict__ proj, long ld, int q_off, int k_off, int v_off,
                                    const float* __restrict__ decay, float* __restrict__ state,
                                    const int* __restrict__ slot_map, const int* __restrict__ q_start,
                                    const int* __restrict__ positions, float* __restrict__ out, long ldo,
                                    int H, int dim, int vd) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dim]
    float* ks = qs + dim;           // [dim]
    __shared__ float part[8][33];
    const int s = blockIdx.x, h = blockIdx.y, v = blockIdx.z * 32 + (threadIdx.x & 31), grp = threadIdx.x >> 5;
    const int t = q_start[s];
    const TP* row = proj + (size_t)t * ld;
    for (int d = threadIdx.x; d < dim; d += 256) {
        qs[d] = silu_f(to_f(row[q_off + (size_t)h * dim + d]));
        ks[d] = silu_f(to_f(row[k_off + (size_t)h * dim + d]));
    }
    __syncthreads();
    float acc = 0.f;
    if (v < vd) {
        const float lam = decay[h];
        const bool fresh = positions[t] == 0;
        const float vv = silu_f(to_f(row[v_off + (size_t)h * vd + v]));
        float* st = state + (((size_t)slot_map[s] * H + h) * dim) * vd + v;
        for (int d0 = grp; d0 < dim; d0 += 32) {                           // four rows' loads in flight
            float sv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) sv[i] = (!fresh && d0 + 8 * i < dim) ? st[(size_t)(d0 + 8 * i) * vd] : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = d0 + 8 * i;
                if (d < dim) {
                    const float n = fmaf(lam, sv[i], ks[d] * vv);
                    st[(size_t)d * vd] = n;
                    acc = fmaf(n, qs[d], acc);
                }
            }
        }
    }
    part[grp][threadIdx.x & 31] = acc;
    __syncthreads();
    if (grp == 0 && v < vd) {
        float o = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) o += part[g][threadIdx.x];
        out[(size_t)t * ldo + (size_t)h * vd + v] = o;
    }
}

// ---------------------------------------------------------------- the same, chunks side by side
// For portions of prompts the chunks of a request need not wait for one another.  Three launches:
//   1. every chunk's own contribution to the state   U_c = sum_j lambda^(n-1-j) k_j v_j^T        (chunks in parallel)
//   2. per request, over its chunks in order          P_c = S (the state before chunk c); S = lambda^n S + U_c
//      (element by element; P_c overwrites U_c in place; the request's slot gets the last S)
//   3. every chunk's outputs                          o_i = sum_{j<=i} (q_i . k_j) lambda^(i-j) v_j + lambda^(i+1) P_c^T q_i
// Chunks of LC tokens are counted from the start of each request's portion; the step has at most T / LC + S of them,
// and a CTA finds its request and chunk from q_start.  All products are float32 on the CUDA cores, in register tiles
// fed from shared memory; a step's result differs from the token-by-token recurrence by rounding only.
constexpr int LC = 64, LVT = 64, LDT = 128, LPAD = 68;

__device__ __forceinline__ bool la_locate(const int* __restrict__ q_start, int S, int c, int& s_out, int& t0, int& n) {
    int acc = 0;
    for (int s = 0; s < S; ++s) {
        const int len = q_start[s + 1] - q_start[s];
        const int nch = (len + LC - 1) / LC;
        if (c < acc + nch) {
            const int k = c - acc;
            s_out = s;
            t0 = q_start[s] + k * LC;
            n = min(LC, len - k * LC);
            return true;
        }
        acc += nch;
    }
    return false;
}

template <typename TP>
__global__ void __launch_bounds__(256)
la_chunk_state_kernel(const TP* __restrict__ proj, long ld, int k_off, int v_off, const float* __restrict__ decay,
                      const int* __restrict__ q_start, int S, float* __restrict__ U, int H, int dim, int vd) {
    __shared__ __align__(16) float Ks[LC][LDT];
    __shared__ __align__(16) float Vs[LC][LVT];
    int s, t0, n;
    const int c = blockIdx.x, h = blockIdx.y;
    if (!la_locate(q_start, S, c, s, t0, n)) return;
    const int vtiles = (vd + LVT - 1) / LVT;
    const int d0 = (blockIdx.z / vtiles) * LDT, v0 = (blockIdx.z % vtiles) * LVT;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float l2 = log2f(decay[h]);
    for (int idx = tid; idx < n * LDT; idx += 256) {
        const int j = idx / LDT, d = idx % LDT;
        float v = 0.f;
        if (d0 + d < dim) v = silu_f(to_f(proj[(size_t)(t0 + j) * ld + k_off + (size_t)h * dim + d0 + d])) * decay_pow(l2, n - 1 - j);
        Ks[j][d] = v;
    }
    for (int idx = tid; idx < n * LVT; idx += 256) {
        const int j = idx / LVT, v = idx % LVT;
        Vs[j][v] = (v0 + v < vd) ? silu_f(to_f(proj[(size_t)(t0 + j) * ld + v_off + (size_t)h * vd + v0 + v])) : 0.f;
    }
    __syncthreads();
    float acc[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    for (int j = 0; j < n; ++j) {
        const float4 ka = *reinterpret_cast<const float4*>(&Ks[j][ty * 8]);
        const float4 kb = *reinterpret_cast<const float4*>(&Ks[j][ty * 8 + 4]);
        const float4 vv = *reinterpret_cast<const float4*>(&Vs[j][tx * 4]);
        const float k8[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
        const float v4[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(k8[a], v4[b], acc[a][b]);
    }
    float* u = U + ((size_t)c * H + h) * dim * vd;
#pragma unroll
    for (int a = 0; a < 8; ++a) {
        const int d = d0 + ty * 8 + a;
        if (d >= dim) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int v = v0 + tx * 4 + b;
            if (v < vd) u[(size_t)d * vd + v] = acc[a][b];
        }
    }
}

__global__ void __launch_bounds__(256)
la_state_scan_kernel(float* __restrict__ U, const float* __restrict__ decay, float* __restrict__ state,
                     const int* __restrict__ slot_map, const int* __restrict__ q_start, const int* __restrict__ positions,
                     int H, int dim, int vd) {
    const int s = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * 256 + threadIdx.x;
    const int E = dim * vd;
    if (e >= E) return;
    int base = 0;
    for (int r = 0; r < s; ++r) base += (q_start[r + 1] - q_start[r] + LC - 1) / LC;
    const int t0 = q_start[s], len = q_start[s + 1] - t0;
    if (len <= 0) return;
    float* st = state + ((size_t)slot_map[s] * H + h) * E + e;
    float Sv = positions[t0] == 0 ? 0.f : *st;
    const float l2 = log2f(decay[h]);
    const float full = decay_pow(l2, LC);
    const int nch = (len + LC - 1) / LC;
    const size_t cstride = (size_t)H * E;
    float* u0 = U + ((size_t)base * H + h) * E + e;
    for (int k0 = 0; k0 < nch; k0 += 8) {                                  // the loads of eight chunks in flight, then their updates in order
        float uv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) uv[i] = (k0 + i < nch) ? __ldcg(u0 + (size_t)(k0 + i) * cstride) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (k0 + i < nch) {
                u0[(size_t)(k0 + i) * cstride] = Sv;
                const int n = min(LC, len - (k0 + i) * LC);
                Sv = fmaf(n == LC ? full : decay_pow(l2, n), Sv, uv[i]);
            }
        }
    }
    *st = Sv;
}

template <typename TP>
__global__ void __launch_bounds__(256)
la_chunk_output_kernel(const TP* __restrict__ proj, long ld, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                       const int* __restrict__ q_start, int S, const float* __restrict__ P, float* __restrict__ out, long ldo,
                       int H, int dim, int vd) {
    extern __shared__ __align__(16) float sm[];
    float* Qt = sm;                         // [dim][LPAD]: Qt[d][i]
    float* Kt = Qt + (size_t)dim * LPAD;    // [dim][LPAD]
    float* At = Kt + (size_t)dim * LPAD;    // [LC][LPAD]: At[j][i]
    float* Vs = At + LC * LPAD;             // [LC][LVT]
    int s, t0, n;
    const int c = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * LVT;
    if (!la_locate(q_start, S, c, s, t0, n)) return;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float l2 = log2f(decay[h]);
    for (int i0 = tid; i0 < LC * dim; i0 += 256 * 8) {                   // eight rows' loads in flight, then their silu and the transposed stores
        float qv[8], kv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = i0 + u * 256;
            const int j = idx / dim, d = idx % dim;
            qv[u] = kv[u] = 0.f;
            if (idx < LC * dim && j < n) {
                const TP* row = proj + (size_t)(t0 + j) * ld + (size_t)h * dim + d;
                qv[u] = to_f(row[q_off]);
                kv[u] = to_f(row[k_off]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = i0 + u * 256;
            if (idx < LC * dim) {
                const int j = idx / dim, d = idx % dim;
                Qt[d * LPAD + j] = j < n ? silu_f(qv[u]) : 0.f;
                Kt[d * LPAD + j] = j < n ? silu_f(kv[u]) : 0.f;
            }
        }
    }
    for (int idx = tid; idx < LC * LVT; idx += 256) {
        const int j = idx / LVT, v = idx % LVT;
        Vs[idx] = (j < n && v0 + v < vd) ? silu_f(to_f(proj[(size_t)(t0 + j) * ld + v_off + (size_t)h * vd + v0 + v])) : 0.f;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    // scores of the chunk: rows i = ty*4.., keys j = tx*4..; tiles wholly above the diagonal stay zero
    if (tx <= ty) {
#pragma unroll 4
        for (int d = 0; d < dim; ++d) {
            const float4 qq = *reinterpret_cast<const float4*>(&Qt[d * LPAD + ty * 4]);
            const float4 kk = *reinterpret_cast<const float4*>(&Kt[d * LPAD + tx * 4]);
            const float q4[4] = {qq.x, qq.y, qq.z, qq.w}, k4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(q4[a], k4[b], acc[a][b]);
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = ty * 4 + a, j = tx * 4 + b;
            At[j * LPAD + i] = (j <= i) ? acc[a][b] * decay_pow(l2, i - j) : 0.f;
        }
    __syncthreads();
    // outputs: rows i = ty*4.., value columns tx*4..
    float o1[4][4], o2[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o1[a][b] = o2[a][b] = 0.f;
    const int jmax = min(n, ty * 4 + 4);
    for (int j = 0; j < jmax; ++j) {
        const float4 aa = *reinterpret_cast<const float4*>(&At[j * LPAD + ty * 4]);
        const float4 vv = *reinterpret_cast<const float4*>(&Vs[j * LVT + tx * 4]);
        const float a4[4] = {aa.x, aa.y, aa.z, aa.w}, v4[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) o1[a][b] = fmaf(a4[a], v4[b], o1[a][b]);
    }
    // the state before the chunk, [dim][LVT] of it, into the space of the keys (used up since the scores)
    {
        const float* p = P + ((size_t)c * H + h) * dim * vd + v0;
        const bool vec = (vd & 3) == 0;
#pragma unroll 4
        for (int idx = tid; idx < dim * (LVT / 4); idx += 256) {
            const int d = idx / (LVT / 4), v4i = (idx % (LVT / 4)) * 4;
            float4 pp = make_float4(0.f, 0.f, 0.f, 0.f);
            if (vec && v0 + v4i + 3 < vd) {
                pp = __ldcg(reinterpret_cast<const float4*>(p + (size_t)d * vd + v4i));
            } else {
                if (v0 + v4i < vd) pp.x = p[(size_t)d * vd + v4i];
                if (v0 + v4i + 1 < vd) pp.y = p[(size_t)d * vd + v4i + 1];
                if (v0 + v4i + 2 < vd) pp.z = p[(size_t)d * vd + v4i + 2];
                if (v0 + v4i + 3 < vd) pp.w = p[(size_t)d * vd + v4i + 3];
            }
            *reinterpret_cast<float4*>(&Kt[d * LPAD + v4i]) = pp;
        }
    }
    __syncthreads();
#pragma unroll 4
    for (int d = 0; d < dim; ++d) {
        const float4 qq = *reinterpret_cast<const float4*>(&Qt[d * LPAD + ty * 4]);
        const float4 pp = *reinterpret_cast<const float4*>(&Kt[d * LPAD + tx * 4]);
        const float q4[4] = {qq.x, qq.y, qq.z, qq.w}, p4[4] = {pp.x, pp.y, pp.z, pp.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) o2[a][b] = fmaf(q4[a], p4[b], o2[a][b]);
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int i = ty * 4 + a;
        if (i >= n) continue;
        const float w = decay_pow(l2, i + 1);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int v = v0 + tx * 4 + b;
            if (v < vd) out[(size_t)(t0 + i) * ldo + (size_t)h * vd + v] = fmaf(w, o2[a][b], o1[a][b]);
        }
    }
}

// out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * w * sigmoid(g[t]): the norm over all heads together, gated.
template <typename TP, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ o, long ldo, const TP* __restrict__ gate, long ldg,
                     const void* __restrict__ w, int wdt, float eps, TO* __restrict__ out, long ldout, int N) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float v = o[t * ldo + i];
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float v = o[t * ldo + i] * scale * load_dyn(w, wdt, i) * sigmoid_f(to_f(gate[t * ldg + i]));
        out[t * ldout + i] = from_f<TO>(v);
    }
}

// ---------------------------------------------------------------- gated recurrence over channels
//   z = sigmoid(pz + bz)    u = px + bx    c = u + 1/2 (u >= 0), sigmoid(u) (u < 0)
//   S_t = (1 - z) S_(t-1) + z c            out_t = S_t * silu(pg)
// One thread per (request, channel) walks the request's portion; neighbouring threads read
// neighbouring channels.  The loads of four tokens are issued before the four dependent updates.
template <typename TP, typename TO>
__global__ void __launch_bounds__(128)
gated_recurrence_kernel(const TP* __restrict__ proj, long ld, int z_off, int x_off, int g_off,
                        const void* __restrict__ bz, const void* __restrict__ bx, int bdt,
                        float* __restrict__ state, const int* __restrict__ slot_map, const int* __restrict__ q_start,
                        const int* __restrict__ positions, TO* __restrict__ out, long ldo, int W) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 <= t0) return;
    float* st = state + (size_t)slot_map[s] * W + c;
    float S = positions[t0] == 0 ? 0.f : *st;
    const float bzc = bz ? load_dyn(bz, bdt, c) : 0.f, bxc = bx ? load_dyn(bx, bdt, c) : 0.f;
    int t = t0;
    for (; t + 4 <= t1; t += 4) {
        float pz[4], px[4], pg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const TP* row = proj + (size_t)(t + i) * ld + c;
            pz[i] = to_f(row[z_off]);
            px[i] = to_f(row[x_off]);
            pg[i] = to_f(row[g_off]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float z = sigmoid_f(pz[i] + bzc), u = px[i] + bxc;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            S = (1.0f - z) * S + z * cand;
            out[(size_t)(t + i) * ldo + c] = from_f<TO>(S * silu_f(pg[i]));
        }
    }
    for (; t < t1; ++t) {
        const TP* row = proj + (size_t)t * ld + c;
        const float z = sigmoid_f(to_f(row[z_off]) + bzc), u = to_f(row[x_off]) + bxc;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = (1.0f - z) * S + z * cand;
        out[(size_t)t * ldo + c] = from_f<TO>(S * silu_f(to_f(row[g_off])));
    }
    *st = S;
}


// The same recurrence for portions of prompts: the portion is cut into GR_SEG segments that run side by side.  A thread
// first reduces its segment to (a, b) with S_end = a S_start + b, the segments' pairs are combined in order through
// shared memory, and the thread walks its segment again from its true starting state, writing the outputs.
constexpr int GR_SEG = 32;

template <typename TP, typename TO>
__global__ void __launch_bounds__(32 * GR_SEG)
gated_recurrence_segments_kernel(const TP* __restrict__ proj, long ld, int z_off, int x_off, int g_off,
                                 const void* __restrict__ bz, const void* __restrict__ bx, int bdt,
                                 float* __restrict__ state, const int* __restrict__ slot_map, const int* __restrict__ q_start,
                                 const int* __restrict__ positions, TO* __restrict__ out, long ldo, int W) {
    __shared__ float As[GR_SEG][33], Bs[GR_SEG][33];
    const int s = blockIdx.y, lane = threadIdx.x, seg = threadIdx.y;
    const int c = blockIdx.x * 32 + lane;
    const bool live = c < W;
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t1 <= t0) return;
    const int per = (t1 - t0 + GR_SEG - 1) / GR_SEG;
    const int lo = min(t1, t0 + seg * per), hi = min(t1, lo + per);
    const float bzc = (live && bz) ? load_dyn(bz, bdt, c) : 0.f, bxc = (live && bx) ? load_dyn(bx, bdt, c) : 0.f;
    float a = 1.f, b = 0.f;
    if (live) {
        for (int t = lo; t < hi; t += 8) {
            float pz[8], px[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const TP* row = proj + (size_t)min(t + i, hi - 1) * ld + c;
                pz[i] = to_f(row[z_off]);
                px[i] = to_f(row[x_off]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (t + i < hi) {
                    const float z = sigmoid_f(pz[i] + bzc), u = px[i] + bxc;
                    const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
                    b = (1.0f - z) * b + z * cand;
                    a *= (1.0f - z);
                }
            }
        }
    }
    As[seg][lane] = a;
    Bs[seg][lane] = b;
    __syncthreads();
    if (!live) return;
    float* st = state + (size_t)slot_map[s] * W + c;
    float Sv = positions[t0] == 0 ? 0.f : *st;
    for (int k = 0; k < seg; ++k) Sv = As[k][lane] * Sv + Bs[k][lane];
    for (int t = lo; t < hi; t += 8) {
        float pz[8], px[8], pg[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const TP* row = proj + (size_t)min(t + i, hi - 1) * ld + c;
            pz[i] = to_f(row[z_off]);
            px[i] = to_f(row[x_off]);
            pg[i] = to_f(row[g_off]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (t + i < hi) {
                const float z = sigmoid_f(pz[i] + bzc), u = px[i] + bxc;
                const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
                Sv = (1.0f - z) * Sv + z * cand;
                out[(size_t)(t + i) * ldo + c] = from_f<TO>(Sv * silu_f(pg[i]));
            }
        }
    }
    if (hi == t1 && lo < hi) *st = Sv;
}

}  // namespace aien

using namespace aien;

static size_t la_smem_bytes(int dim) {
    return (size_t)(2 * LA_C * (dim + 1) + LA_C * LA_VS + LA_C * (LA_C + 1) + dim * LA_VS) * sizeof(float);
}

template <typename TP>
static int launch_decay_linear_attention(int single_tokens, dim3 grid, size_t smem, cudaStream_t stream, const TP* proj, long ld, int q_off, int k_off,
                                         int v_off, const float* decay, float* state, const int* slot_map, const int* q_start,
                                         const int* positions, float* out, long ldo, int H, int dim, int vd) {
    if (single_tokens) {
        decay_linear_attention_token_kernel<TP><<<dim3(grid.x, grid.y, (vd + 31) / 32), 256, 2 * dim * sizeof(float), stream>>>(
            proj, ld, q_off, k_off, v_off, decay, state, slot_map, q_start, positions, out, ldo, H, dim, vd);
        return 0;
    }
    auto kern = decay_linear_attention_kernel<TP>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<grid, LA_THREADS, smem, stream>>>(proj, ld, q_off, k_off, v_off, decay, state, slot_map, q_start, positions, out, ldo, H, dim, vd);
    return 0;
}

// proj [T, ld]: the projections before their silu, q at column q_off (H*dim), k at k_off, v at v_off (H*vd).
// decay float32 [H]; state float32 [slots, H, dim, vd]; out float32 [T, ldo] receives o (H*vd per token).
// single_tokens != 0: every request of the step brings exactly one token (the state streams through once).
AIEN_API int aien_decay_linear_attention(const void* proj, int p_dt, long ld, int q_off, int k_off, int v_off,
                                         const float* decay, float* state, const int* slot_map, const int* q_start,
                                         const int* positions, float* out, long ldo, int S, int H, int dim, int vd,
                                         int single_tokens, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H <= 0 || dim <= 0 || vd <= 0 || H > 65535) return AIEN_E_SHAPE;
    const size_t smem = la_smem_bytes(dim);
    if (smem > 200 * 1024) return AIEN_E_SHAPE;
    dim3 grid(S, H, (vd + LA_VS - 1) / LA_VS);
    if (grid.z > 65535) return AIEN_E_SHAPE;
    int rc = 0;
    AIEN_DISPATCH_DTYPE(p_dt, TP, (rc = launch_decay_linear_attention<TP>(single_tokens, grid, smem, stream, (const TP*)proj, ld, q_off, k_off, v_off, decay,
                                                                          state, slot_map, q_start, positions, out, ldo, H, dim, vd)));
    if (rc != 0) return rc;
    return launch_status();
}

template <typename TP>
static int launch_la_chunked(cudaStream_t stream, const TP* proj, long ld, int q_off, int k_off, int v_off, const float* decay,
                             float* state, const int* slot_map, const int* q_start, const int* positions, float* out, long ldo,
                             float* U, int T, int S, int H, int dim, int vd) {
    const int NC = T / LC + S;
    const int dtiles = (dim + LDT - 1) / LDT, vtiles = (vd + LVT - 1) / LVT;
    const size_t smem = ((size_t)2 * dim * LPAD + LC * LPAD + LC * LVT) * sizeof(float);
    auto kout = la_chunk_output_kernel<TP>;
    if (smem > 200 * 1024) return AIEN_E_SHAPE;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kout, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    la_chunk_state_kernel<TP><<<dim3(NC, H, dtiles * vtiles), 256, 0, stream>>>(proj, ld, k_off, v_off, decay, q_start, S, U, H, dim, vd);
    la_state_scan_kernel<<<dim3((dim * vd + 255) / 256, H, S), 256, 0, stream>>>(U, decay, state, slot_map, q_start, positions, H, dim, vd);
    kout<<<dim3(NC, H, vtiles), 256, smem, stream>>>(proj, ld, q_off, k_off, v_off, decay, q_start, S, U, out, ldo, H, dim, vd);
    return 0;
}

// The same result as aien_decay_linear_attention for a step of T tokens in S requests, chunks side by side.
// scratch: float32, (T / 64 + S) * H * dim * vd numbers.
AIEN_API int aien_decay_linear_attention_chunked(const void* proj, int p_dt, long ld, int q_off, int k_off, int v_off,
                                                 const float* decay, float* state, const int* slot_map, const int* q_start,
                                                 const int* positions, float* out, long ldo, float* scratch, int T, int S,
                                                 int H, int dim, int vd, cudaStream_t stream) {
    if (S <= 0 || T <= 0) return 0;
    if (H <= 0 || dim <= 0 || vd <= 0 || H > 65535 || S > 65535 || scratch == nullptr) return AIEN_E_SHAPE;
    int rc = 0;
    AIEN_DISPATCH_DTYPE(p_dt, TP, (rc = launch_la_chunked<TP>(stream, (const TP*)proj, ld, q_off, k_off, v_off, decay, state, slot_map,
                                                              q_start, positions, out, ldo, scratch, T, S, H, dim, vd)));
    if (rc != 0) return rc;
    return launch_status();
}

AIEN_API int aien_gated_rmsnorm(const float* o, long ldo, const void* gate, int g_dt, long ldg, const void* w, int w_dt, float eps,
                                void* out, int o_dt, long ldout, int T, int N, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N <= 0) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(g_dt, TP, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (gated_rmsnorm_kernel<TP, TO><<<T, 256, 0, stream>>>(o, ldo, (const TP*)gate, ldg, w, w_dt, eps, (TO*)out, ldout, N))));
    return launch_status();
}

// proj [T, ld]: z at column z_off, the candidate's input at x_off, the output gate at g_off (W each); bz, bx [W] or null.
// state float32 [slots, W]; out [T, ldo] in its own dtype.  segments != 0: every portion is cut into segments that run side by side.
AIEN_API int aien_gated_recurrence(const void* proj, int p_dt, long ld, int z_off, int x_off, int g_off,
                                   const void* bz, const void* bx, int b_dt, float* state, const int* slot_map,
                                   const int* q_start, const int* positions, void* out, int o_dt, long ldo,
                                   int S, int W, int segments, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (W <= 0 || S > 65535) return AIEN_E_SHAPE;
    if (segments) {
        AIEN_DISPATCH_DTYPE(p_dt, TP, AIEN_DISPATCH_DTYPE(o_dt, TO,
            (gated_recurrence_segments_kernel<TP, TO><<<dim3((W + 31) / 32, S), dim3(32, GR_SEG), 0, stream>>>(
                (const TP*)proj, ld, z_off, x_off, g_off, bz, bx, b_dt, state, slot_map, q_start, positions, (TO*)out, ldo, W))));
        return launch_status();
    }
    dim3 grid((W + 127) / 128, S);
    AIEN_DISPATCH_DTYPE(p_dt, TP, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (gated_recurrence_kernel<TP, TO><<<grid, 128, 0, stream>>>((const TP*)proj, ld, z_off, x_off, g_off, bz, bx, b_dt, state,
                                                                  slot_map, q_start, positions, (TO*)out, ldo, W))));
    return launch_status();
}
