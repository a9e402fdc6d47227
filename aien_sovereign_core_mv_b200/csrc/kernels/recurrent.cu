// Recurrent mixers whose state has a fixed size per request: linear attention with a per-head
// decay, and a gated recurrence over channels.  The state is float32 and lives in a state slot
// of the cache ([slots, ...]); everything that enters a recurrence (decay powers, gates,
// candidates, the state itself, the products with it) is float32 in both engine precisions.
//
// The contract of a state slot, all of it on the device: the portion of request s of the step is
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

}  // namespace aien

using namespace aien;

static size_t la_smem_bytes(int dim) {
    return (size_t)(2 * LA_C * (dim + 1) + LA_C * LA_VS + LA_C * (LA_C + 1) + dim * LA_VS) * sizeof(float);
}

template <typename TP>
static int launch_decay_linear_attention(dim3 grid, size_t smem, cudaStream_t stream, const TP* proj, long ld, int q_off, int k_off,
                                         int v_off, const float* decay, float* state, const int* slot_map, const int* q_start,
                                         const int* positions, float* out, long ldo, int H, int dim, int vd) {
    auto kern = decay_linear_attention_kernel<TP>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<grid, LA_THREADS, smem, stream>>>(proj, ld, q_off, k_off, v_off, decay, state, slot_map, q_start, positions, out, ldo, H, dim, vd);
    return 0;
}

// proj [T, ld]: the projections before their silu, q at column q_off (H*dim), k at k_off, v at v_off (H*vd).
// decay float32 [H]; state float32 [slots, H, dim, vd]; out float32 [T, ldo] receives o (H*vd per token).
AIEN_API int aien_decay_linear_attention(const void* proj, int p_dt, long ld, int q_off, int k_off, int v_off,
                                         const float* decay, float* state, const int* slot_map, const int* q_start,
                                         const int* positions, float* out, long ldo, int S, int H, int dim, int vd,
                                         cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H <= 0 || dim <= 0 || vd <= 0 || H > 65535) return AIEN_E_SHAPE;
    const size_t smem = la_smem_bytes(dim);
    if (smem > 200 * 1024) return AIEN_E_SHAPE;
    dim3 grid(S, H, (vd + LA_VS - 1) / LA_VS);
    if (grid.z > 65535) return AIEN_E_SHAPE;
    int rc = 0;
    AIEN_DISPATCH_DTYPE(p_dt, TP, (rc = launch_decay_linear_attention<TP>(grid, smem, stream, (const TP*)proj, ld, q_off, k_off, v_off, decay,
                                                                          state, slot_map, q_start, positions, out, ldo, H, dim, vd)));
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
// state float32 [slots, W]; out [T, ldo] in its own dtype.
AIEN_API int aien_gated_recurrence(const void* proj, int p_dt, long ld, int z_off, int x_off, int g_off,
                                   const void* bz, const void* bx, int b_dt, float* state, const int* slot_map,
                                   const int* q_start, const int* positions, void* out, int o_dt, long ldo,
                                   int S, int W, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (W <= 0 || S > 65535) return AIEN_E_SHAPE;
    dim3 grid((W + 127) / 128, S);
    AIEN_DISPATCH_DTYPE(p_dt, TP, AIEN_DISPATCH_DTYPE(o_dt, TO,
        (gated_recurrence_kernel<TP, TO><<<grid, 128, 0, stream>>>((const TP*)proj, ld, z_off, x_off, g_off, bz, bx, b_dt, state,
                                                                  slot_map, q_start, positions, (TO*)out, ldo, W))));
    return launch_status();
}
