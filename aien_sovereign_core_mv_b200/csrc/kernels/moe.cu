// Routed feed-forward: the router's choice and the plain expert products.
//
//   route        scores s = softmax(z) over all E experts (float32); experts lie in `groups` equal
//                groups of neighbours, a group scores its best expert, only the `keep` best groups
//                stay eligible; the `top` best eligible experts are taken, weight = their score
//                (divided by the sum of the taken scores when `renorm` is set).  Ties go to the lower
//                index.  One warp per token.
//   expert_up    act[t, c, :] = f(W_up[e(t,c)] h[t])             c < top, f = gelu (erf or tanh form)
//   expert_down  part[c][t, :] = weight(t,c) * W_down[e(t,c)] act[t, c, :]   float32 parts, one per choice,
//                which the consumer (the norm that takes the branch) adds in index order
//   act_rows     f applied in place to [T, F] rows (the shared expert's hidden layer)
//
// The products here are one warp per output value with the reduction in a fixed lane order, so a
// token's result depends on its own row alone; they serve the 32-bit engine and small steps, and
// are what the grouped tensor-core products are held to.
#include "common.cuh"
#include <math.h>

namespace aien {

__device__ __forceinline__ float act_apply(float z, int kind) {
    if (kind == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
}

// ---------------------------------------------------------------- router
constexpr int ROUTE_MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(32)
moe_route_kernel(const float* __restrict__ z, int E, int groups, int keep, int top, int renorm,
                 int* __restrict__ ids, float* __restrict__ wts) {
    __shared__ float s[ROUTE_MAX_EXPERTS];
    __shared__ float gs[ROUTE_MAX_EXPERTS];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* zr = z + (size_t)t * E;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) { const float v = __ldcg(zr + e); s[e] = v; m = fmaxf(m, v); }
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - m); s[e] = v; sum += v; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) s[e] *= inv;
    __syncwarp();
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int j = 0; j < per; ++j) best = fmaxf(best, s[g * per + j]);
            gs[g] = best;
        }
        __syncwarp();
        // every group starts ineligible (score negated below zero); the `keep` best are restored
        for (int r = 0; r < keep; ++r) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) if (gs[g] > bv) { bv = gs[g]; bi = g; }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) gs[bi] = -1.0f;                 // marks a kept group (scores are >= 0)
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (gs[e / per] != -1.0f) s[e] = -1.0f;      // not eligible
        __syncwarp();
    }
    float wsum = 0.f;
    for (int r = 0; r < top; ++r) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) if (s[e] > bv) { bv = s[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            ids[(size_t)t * top + r] = bi;
            wts[(size_t)t * top + r] = bv;
            s[bi] = -2.0f;                                 // taken
        }
        wsum += bv;
        __syncwarp();
    }
    if (renorm && lane == 0) {
        for (int r = 0; r < top; ++r) wts[(size_t)t * top + r] /= wsum;
    }
}

// ---------------------------------------------------------------- plain expert products
// One warp per output value; 8 warps a CTA take 8 consecutive output rows of one (token, choice).
template <typename TH, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_expert_up_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w_up, const int* __restrict__ ids,
                     TO* __restrict__ act, int top, int D, int F, int act_kind) {
    griddep_launch();
    griddep_wait();
    const int pair = blockIdx.x;                       // t * top + c
    const int t = pair / top;
    const int f = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (f >= F) return;
    const int e = __ldcg(ids + pair);
    const TW* wr = w_up + ((size_t)e * F + f) * D;
    const TH* hr = h + (size_t)t * h_stride;
    float acc = 0.f;
    for (int i = lane; i < D; i += 32) acc = fmaf(to_f(wr[i]), ld_act(hr + i), acc);
    acc = warp_sum(acc);
    if (lane == 0) act[(size_t)pair * F + f] = from_f<TO>(act_apply(acc, act_kind));
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
moe_expert_down_kernel(const TA* __restrict__ act, const TW* __restrict__ w_down, const int* __restrict__ ids,
                       const float* __restrict__ wts, float* __restrict__ parts, int T, int top, int D, int F) {
    griddep_launch();
    griddep_wait();
    const int pair = blockIdx.x;
    const int t = pair / top, c = pair - t * top;
    const int n = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= D) return;
    const int e = __ldcg(ids + pair);
    const TW* wr = w_down + ((size_t)e * D + n) * F;
    const TA* ar = act + (size_t)pair * F;
    float acc = 0.f;
    for (int i = lane; i < F; i += 32) acc = fmaf(to_f(wr[i]), ld_act(ar + i), acc);
    acc = warp_sum(acc);
    if (lane == 0) parts[((size_t)c * T + t) * D + n] = acc * __ldcg(wts + pair);
}

template <typename T>
__global__ void act_rows_kernel(T* __restrict__ a, size_t n, int act_kind) {
    griddep_launch();
    griddep_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        a[i] = from_f<T>(act_apply(ld_act(a + i), act_kind));
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_moe_route(const float* z, int T, int E, int groups, int keep, int top, int renorm, int* ids, float* wts,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > ROUTE_MAX_EXPERTS || groups <= 0 || E % groups != 0 || keep <= 0 || keep > groups || top <= 0 ||
        top > keep * (E / groups)) return AIEN_E_SHAPE;
    launch_chain(moe_route_kernel, dim3(T), dim3(32), 0, stream, z, E, groups, keep, top, renorm, ids, wts);
    return launch_status();
}

// h [T, D] (row stride h_stride), w_up [E, F, D], act [T * top, F]; act_kind 0: erf gelu, 1: tanh gelu.
AIEN_API int aien_moe_expert_up(const void* h, int h_dt, long h_stride, const void* w_up, int w_dt, const int* ids,
                                void* act, int act_dt, int T, int top, int D, int F, int act_kind, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T * (long)top > 2147483647L || D <= 0 || F <= 0 || (F + 7) / 8 > 65535) return AIEN_E_SHAPE;
    dim3 grid(T * top, (F + 7) / 8);
    AIEN_DISPATCH_DTYPE(h_dt, TH, AIEN_DISPATCH_DTYPE(w_dt, TW, AIEN_DISPATCH_DTYPE(act_dt, TO,
        (launch_chain(moe_expert_up_kernel<TH, TW, TO>, grid, dim3(256), 0, stream,
                      (const TH*)h, h_stride, (const TW*)w_up, ids, (TO*)act, top, D, F, act_kind)))));
    return launch_status();
}

// act [T * top, F], w_down [E, D, F], parts float32 [top, T, D].
AIEN_API int aien_moe_expert_down(const void* act, int act_dt, const void* w_down, int w_dt, const int* ids, const float* wts,
                                  float* parts, int T, int top, int D, int F, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T * (long)top > 2147483647L || D <= 0 || F <= 0 || (D + 7) / 8 > 65535) return AIEN_E_SHAPE;
    dim3 grid(T * top, (D + 7) / 8);
    AIEN_DISPATCH_DTYPE(act_dt, TA, AIEN_DISPATCH_DTYPE(w_dt, TW,
        (launch_chain(moe_expert_down_kernel<TA, TW>, grid, dim3(256), 0, stream,
                      (const TA*)act, (const TW*)w_down, ids, wts, parts, T, top, D, F))));
    return launch_status();
}

AIEN_API int aien_act_rows(void* a, int dt, size_t n, int act_kind, cudaStream_t stream) {
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    AIEN_DISPATCH_DTYPE(dt, TT, (launch_chain(act_rows_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (TT*)a, n, act_kind)));
    return launch_status();
}
