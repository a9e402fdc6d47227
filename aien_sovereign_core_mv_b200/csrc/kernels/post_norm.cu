// Pieces of a layer that norms a sublayer's input and its output:
//
//     x[t] += mult * y[t] / sqrt(mean(y[t]^2) + eps) * w          y[t] = sum_p a[p][t]
//     h[t]  = x[t] / sqrt(mean(x[t]^2) + eps_next) * w_next        (or the plain copy of x[t], or nothing)
//
// in one pass over the row: the norm of the branch's output, its scaled sum into the float32 stream, and
// the norm that the next sublayer reads.  Both sums of squares, both scales and the sum are float32.
// One CTA per row; the row stays in shared memory between the passes.  Also here: the embedding row
// times a constant, gelu(z) * (a slice of a second embedding row), and the soft cap of logits.
#include "common.cuh"
#include <math.h>

namespace aien {

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TA, typename TH>
__global__ void __launch_bounds__(256)
post_norm_add_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_parts, size_t a_stride,
                     const void* __restrict__ w, int wdt, float eps, float mult,
                     const void* __restrict__ w_next, int wndt, float eps_next, TH* __restrict__ h, int H) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = 0.f;
        for (int p = 0; p < a_parts; ++p) v += to_f(a[(size_t)p * a_stride + base + i]);
        row[i] = v;
        ss += v * v;
    }
    const float scale = mult / sqrtf(block_sum(ss, red) / (float)H + eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float r = x[base + i] + row[i] * scale * load_dyn(w, wdt, i);
        x[base + i] = r;
        row[i] = r;
        ss2 += r * r;
    }
    if (h == nullptr) return;
    if (w_next == nullptr) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) h[base + i] = from_f<TH>(row[i]);
        return;
    }
    const float scale2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)H + eps_next);
    for (int i = threadIdx.x; i < H; i += blockDim.x) h[base + i] = from_f<TH>(row[i] * scale2 * load_dyn(w_next, wndt, i));
}


// The same for rows of whole float4 vectors (H % 4 == 0, 16-byte aligned rows): every thread owns up to NV vectors of
// the row and keeps them in registers between the passes, with all loads of a pass in flight at once; the CTA has as
// many threads as the row has vectors (up to 512).  Parts are added in the order of the plain kernel; which of the two
// kernels a row takes follows from H and the pointers alone, never from the step.
__device__ __forceinline__ float4 pn_w4(const void* w, int wdt, int v) {
    if (wdt == AIEN_DT_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + 4 * v);
    return ld_act4(reinterpret_cast<const __nv_bfloat16*>(w) + 4 * v);
}
__device__ __forceinline__ void pn_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void pn_store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename TA, typename TH, int NV>
__global__ void __launch_bounds__(512)
post_norm_add_vec_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_parts, size_t a_stride,
                         const void* __restrict__ w, int wdt, float eps, float mult,
                         const void* __restrict__ w_next, int wndt, float eps_next, TH* __restrict__ h, int H) {
    __shared__ float red[32];
    const int nvec = H >> 2;
    const size_t base = (size_t)blockIdx.x * H;
    float4 y[NV], xv[NV], wv[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        y[j] = xv[j] = wv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (v < nvec) {
            wv[j] = pn_w4(w, wdt, v);
            xv[j] = *reinterpret_cast<const float4*>(x + base + 4 * (size_t)v);
            for (int p = 0; p < a_parts; ++p) {
                const float4 t = ld_act4(a + (size_t)p * a_stride + base + 4 * (size_t)v);
                y[j].x += t.x; y[j].y += t.y; y[j].z += t.z; y[j].w += t.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) ss += y[j].x * y[j].x + y[j].y * y[j].y + y[j].z * y[j].z + y[j].w * y[j].w;
    const float scale = mult / sqrtf(block_sum(ss, red) / (float)H + eps);
    float ss2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        xv[j] = make_float4(xv[j].x + y[j].x * scale * wv[j].x, xv[j].y + y[j].y * scale * wv[j].y,
                            xv[j].z + y[j].z * scale * wv[j].z, xv[j].w + y[j].w * scale * wv[j].w);
        if (v < nvec) {
            *reinterpret_cast<float4*>(x + base + 4 * (size_t)v) = xv[j];
            ss2 += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
        }
    }
    if (h == nullptr) return;
    if (w_next == nullptr) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) pn_store4(h + base + 4 * (size_t)v, xv[j]);
        }
        return;
    }
    const float scale2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)H + eps_next);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) {
            const float4 n = pn_w4(w_next, wndt, v);
            pn_store4(h + base + 4 * (size_t)v, make_float4(xv[j].x * scale2 * n.x, xv[j].y * scale2 * n.y, xv[j].z * scale2 * n.z, xv[j].w * scale2 * n.w));
        }
    }
}

template <typename TW>
__global__ void embed_gather_scaled_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                                           int H, int V, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* row = x + (size_t)t * H;
    if (id < 0 || id >= V) {                      // refused on the host; never read out of range
        for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = to_f(src[i]) * scale;
}

// g[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j], j < n
template <typename TZ, typename TW, typename TO>
__global__ void gelu_times_table_kernel(const TZ* __restrict__ z, long ldz, const TW* __restrict__ table, long ldt, int col0,
                                        const int* __restrict__ ids, int V, TO* __restrict__ g, long ldg, int n) {
    const size_t t = blockIdx.x;
    const int id = ids[t];
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float e = (id >= 0 && id < V) ? to_f(table[(size_t)id * ldt + col0 + j]) : 0.f;
        g[t * ldg + j] = from_f<TO>(gelu_tanh_f(to_f(z[t * ldz + j])) * e);
    }
}

__global__ void softcap_kernel(float* __restrict__ v, size_t n, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = cap * tanhf(v[i] / cap);
}

}  // namespace aien

using namespace aien;

template <typename TA, typename TH>
static int launch_post_norm_add(size_t smem, cudaStream_t stream, float* x, const TA* a, int a_parts, size_t a_stride, const void* w,
                                int w_dt, float eps, float mult, const void* w_next, int wn_dt, float eps_next, TH* h, int T, int H) {
    {
        const int nvec = H >> 2;
        const int threads = nvec >= 512 ? 512 : ((nvec + 31) & ~31);
        const int wsz = w_dt == AIEN_DT_F32 ? 15 : 7, wnsz = wn_dt == AIEN_DT_F32 ? 15 : 7, asz = sizeof(TA) == 4 ? 15 : 7, hsz = sizeof(TH) == 4 ? 15 : 7;
        const bool aligned = (H & 3) == 0 && threads > 0 && nvec <= threads * 4 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)a & asz) == 0 &&
                             ((uintptr_t)w & wsz) == 0 && ((uintptr_t)w_next & wnsz) == 0 && ((uintptr_t)h & hsz) == 0 && (a_stride & 3) == 0;
        if (aligned) {
            if (nvec <= threads)
                post_norm_add_vec_kernel<TA, TH, 1><<<T, threads, 0, stream>>>(x, a, a_parts, a_stride, w, w_dt, eps, mult, w_next, wn_dt, eps_next, h, H);
            else if (nvec <= 2 * threads)
                post_norm_add_vec_kernel<TA, TH, 2><<<T, threads, 0, stream>>>(x, a, a_parts, a_stride, w, w_dt, eps, mult, w_next, wn_dt, eps_next, h, H);
            else
                post_norm_add_vec_kernel<TA, TH, 4><<<T, threads, 0, stream>>>(x, a, a_parts, a_stride, w, w_dt, eps, mult, w_next, wn_dt, eps_next, h, H);
            return 0;
        }
    }
    auto kern = post_norm_add_kernel<TA, TH>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return AIEN_E_STATE;
    kern<<<T, 256, smem, stream>>>(x, a, a_parts, a_stride, w, w_dt, eps, mult, w_next, wn_dt, eps_next, h, H);
    return 0;
}

// a: [T,H] in a_dt, or a_parts float32 parts a_stride apart.  w_next null: h (if given) receives the plain copy of the new row.
AIEN_API int aien_post_norm_add(float* x, const void* a, int a_dt, int a_parts, size_t a_stride, const void* w, int w_dt, float eps,
                                float mult, const void* w_next, int wn_dt, float eps_next, void* h, int h_dt, int T, int H,
                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || a == nullptr || a_parts < 1 || (size_t)H * 4 > 160 * 1024) return AIEN_E_SHAPE;
    const size_t smem = (size_t)H * sizeof(float);
    int rc = 0;
    AIEN_DISPATCH_DTYPE(a_dt, TA, AIEN_DISPATCH_DTYPE(h_dt, TH,
        (rc = launch_post_norm_add<TA, TH>(smem, stream, x, (const TA*)a, a_parts, a_stride, w, w_dt, eps, mult, w_next, wn_dt, eps_next,
                                           (TH*)h, T, H))));
    if (rc != 0) return rc;
    return launch_status();
}

AIEN_API int aien_embed_gather_scaled(const void* table, int table_dt, const int* ids, float* x, int T, int H, int V, float scale,
                                      cudaStream_t stream) {
    if (T <= 0) return 0;
    AIEN_DISPATCH_DTYPE(table_dt, TW, (embed_gather_scaled_kernel<TW><<<T, 256, 0, stream>>>((const TW*)table, ids, x, H, V, scale)));
    return launch_status();
}

AIEN_API int aien_gelu_times_table(const void* z, int z_dt, long ldz, const void* table, int t_dt, long ldt, int col0, const int* ids,
                                   int V, void* g, int g_dt, long ldg, int T, int n, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    AIEN_DISPATCH_DTYPE(z_dt, TZ, AIEN_DISPATCH_DTYPE(t_dt, TW, AIEN_DISPATCH_DTYPE(g_dt, TO,
        (gelu_times_table_kernel<TZ, TW, TO><<<T, 128, 0, stream>>>((const TZ*)z, ldz, (const TW*)table, ldt, col0, ids, V, (TO*)g, ldg, n)))));
    return launch_status();
}

AIEN_API int aien_softcap(float* v, size_t n, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    if (!(cap > 0.f)) return AIEN_E_SHAPE;
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(v, n, cap);
    return launch_status();
}
