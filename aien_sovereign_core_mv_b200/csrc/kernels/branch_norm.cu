// The norm of a residual branch's *output*, added into the stream:
//
//     x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w        y[t] = sum_p a[p][t] + sum_p b[p][t]
//
// for blocks that norm what a sublayer returns instead of what it reads.  The branch output may
// come as one tensor or as float32 partial products (a product cut over K, or the weighted
// outputs of routed experts, one part per choice) and as two such sources (routed parts plus a
// shared expert); parts are added in index order, `a` before `b`.  The sum of squares, the scale
// and the sum into x are float32.  `h` (optional) receives the updated row in the compute dtype:
// the next sublayer reads x itself, so the copy it multiplies by is made here and not by a pass
// of its own.  One CTA per row; the weight vector is the effective one (an offset already added).
#include "common.cuh"

namespace aien {

template <typename T>
__device__ __forceinline__ float parts_sum(const T* __restrict__ p, int nparts, size_t part_stride, size_t idx) {
    float d = 0.f;
    for (int i = 0; i < nparts; ++i) d += ld_act(p + (size_t)i * part_stride + idx);
    return d;
}

constexpr int BN_THREADS = 256;
constexpr int BN_KEEP = 8;        // values of the row a thread keeps in registers between the passes

template <typename TA, typename TB, typename TH>
__global__ void __launch_bounds__(BN_THREADS)
branch_norm_add_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_parts, size_t a_stride,
                       const TB* __restrict__ b, int b_parts, size_t b_stride,
                       const void* __restrict__ w, int wdt, float eps, TH* __restrict__ h, int H) {
    __shared__ float red[32];
    griddep_launch();
    griddep_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float keep[BN_KEEP];
    float ss = 0.f;
    int n = 0;
    for (int i = threadIdx.x; i < H; i += BN_THREADS, ++n) {
        float v = parts_sum(a, a_parts, a_stride, base + i);
        if (b != nullptr) v += parts_sum(b, b_parts, b_stride, base + i);
        if (n < BN_KEEP) keep[n] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)H + eps);
    n = 0;
    for (int i = threadIdx.x; i < H; i += BN_THREADS, ++n) {
        float v;
        if (n < BN_KEEP) {
            v = keep[n];
        } else {                                           // rows wider than 2,048: summed again, same order, same bits
            v = parts_sum(a, a_parts, a_stride, base + i);
            if (b != nullptr) v += parts_sum(b, b_parts, b_stride, base + i);
        }
        const float r = x[base + i] + v * scale * load_dyn(w, wdt, i);
        x[base + i] = r;
        if (h != nullptr) h[base + i] = from_f<TH>(r);
    }
}

// The same for rows of whole float4 vectors (H % 4 == 0, 16-byte aligned rows): every thread owns up
// to BN_VECS vectors of the row, keeps their sums in registers between the passes, and has all the
// loads of a pass in flight at once; the CTA has as many threads as the row has vectors (up to 512),
// so a step of few rows still spreads a row's loads over many threads.  Parts are added in the order
// of the plain kernel above; the sum of squares has a fixed order of its own.  Which of the two
// kernels a row takes follows from H alone, never from the step.
constexpr int BN_VECS = 4;        // at most; a row of up to 512 / 1,024 vectors takes the kernel made for 1 / 2 (fewer registers, more CTAs an SM)

__device__ __forceinline__ float4 f4_add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

template <typename T>
__device__ __forceinline__ float4 parts_sum4(const T* __restrict__ p, int nparts, size_t part_stride, size_t idx) {
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int i = 0; i < nparts; ++i) d = f4_add(d, ld_act4(p + (size_t)i * part_stride + idx));
    return d;
}

__device__ __forceinline__ void store_h4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store_h4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename TA, typename TB, typename TH, int NV>
__global__ void __launch_bounds__(512)
branch_norm_add_vec_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_parts, size_t a_stride,
                           const TB* __restrict__ b, int b_parts, size_t b_stride,
                           const float* __restrict__ w, float eps, TH* __restrict__ h, int H) {
    __shared__ float red[32];
    griddep_launch();
    const int nvec = H >> 2;
    float4 wv[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {                                   // the weights do not depend on the kernel ahead
        const int v = threadIdx.x + j * blockDim.x;
        wv[j] = v < nvec ? *reinterpret_cast<const float4*>(w + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    griddep_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float4 y[NV], xv[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        y[j] = xv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (v < nvec) {
            xv[j] = __ldcg(reinterpret_cast<const float4*>(x + base) + v);
            y[j] = parts_sum4(a, a_parts, a_stride, base + 4 * (size_t)v);
            if (b != nullptr) y[j] = f4_add(y[j], parts_sum4(b, b_parts, b_stride, base + 4 * (size_t)v));
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) ss += y[j].x * y[j].x + y[j].y * y[j].y + y[j].z * y[j].z + y[j].w * y[j].w;
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) {
            const float4 r = make_float4(xv[j].x + y[j].x * scale * wv[j].x, xv[j].y + y[j].y * scale * wv[j].y,
                                         xv[j].z + y[j].z * scale * wv[j].z, xv[j].w + y[j].w * scale * wv[j].w);
            *reinterpret_cast<float4*>(x + base + 4 * (size_t)v) = r;
            if (h != nullptr) store_h4(h + base + 4 * (size_t)v, r);
        }
    }
}

// x[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w in place (the norm of the embedding row), h as above.
template <typename TH>
__global__ void __launch_bounds__(BN_THREADS)
stream_norm_inplace_kernel(float* __restrict__ x, const void* __restrict__ w, int wdt, float eps, TH* __restrict__ h, int H) {
    __shared__ float red[32];
    griddep_launch();
    griddep_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += BN_THREADS) {
        const float v = __ldcg(x + base + i);
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += BN_THREADS) {
        const float r = __ldcg(x + base + i) * scale * load_dyn(w, wdt, i);
        x[base + i] = r;
        if (h != nullptr) h[base + i] = from_f<TH>(r);
    }
}

}  // namespace aien

using namespace aien;

// a_dt / b_dt: dtype of the sources (parts of either dtype are added in float32); h_dt: dtype of h.
AIEN_API int aien_branch_norm_add(float* x, const void* a, int a_dt, int a_parts, size_t a_stride,
                                  const void* b, int b_dt, int b_parts, size_t b_stride,
                                  const void* w, int w_dt, float eps, void* h, int h_dt, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || a == nullptr || a_parts < 1 || (b != nullptr && b_parts < 1)) return AIEN_E_SHAPE;
    {
        const int nvec = H >> 2;
        const int threads = nvec >= 512 ? 512 : ((nvec + 31) & ~31);
        const bool aligned = (H & 3) == 0 && w_dt == AIEN_DT_F32 && threads > 0 && nvec <= threads * BN_VECS &&
                             (((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w | (uintptr_t)h) & 15) == 0 &&
                             (a_stride & 3) == 0 && (b_stride & 3) == 0 &&
                             (a_dt == AIEN_DT_F32 || ((uintptr_t)a & 7) == 0) && (b == nullptr || b_dt == AIEN_DT_F32 || ((uintptr_t)b & 7) == 0);
        if (aligned) {
#define BN_LAUNCH(NVV)                                                                                                          \
            AIEN_DISPATCH_DTYPE(a_dt, TA, AIEN_DISPATCH_DTYPE(b_dt, TB, AIEN_DISPATCH_DTYPE(h_dt, TH,                               \
                (launch_chain(branch_norm_add_vec_kernel<TA, TB, TH, NVV>, dim3(T), dim3(threads), 0, stream,                        \
                              x, (const TA*)a, a_parts, a_stride, (const TB*)b, b_parts, b_stride, (const float*)w, eps, (TH*)h, H)))))
            if (nvec <= threads) { BN_LAUNCH(1); }
            else if (nvec <= 2 * threads) { BN_LAUNCH(2); }
            else { BN_LAUNCH(4); }
#undef BN_LAUNCH
            return launch_status();
        }
    }
    AIEN_DISPATCH_DTYPE(a_dt, TA, AIEN_DISPATCH_DTYPE(b_dt, TB, AIEN_DISPATCH_DTYPE(h_dt, TH,
        (launch_chain(branch_norm_add_kernel<TA, TB, TH>, dim3(T), dim3(BN_THREADS), 0, stream,
                      x, (const TA*)a, a_parts, a_stride, (const TB*)b, b_parts, b_stride, w, w_dt, eps, (TH*)h, H)))));
    return launch_status();
}

AIEN_API int aien_stream_norm_inplace(float* x, const void* w, int w_dt, float eps, void* h, int h_dt, int T, int H,
                                      cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(h_dt, TH,
        (launch_chain(stream_norm_inplace_kernel<TH>, dim3(T), dim3(BN_THREADS), 0, stream, x, w, w_dt, eps, (TH*)h, H)));
    return launch_status();
}
