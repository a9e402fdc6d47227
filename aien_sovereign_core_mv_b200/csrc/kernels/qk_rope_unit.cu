// q/k preparation for attention whose rotation pairs neighbouring dimensions and whose q and k
// are brought to unit root-mean-square *after* the rotation, with the values taken from the key
// projection itself:
//
//   pair i of a head = dimensions (2i, 2i+1), i < rot/2:  (a, b) -> (a cos - b sin, b cos + a sin)
//   with cos/sin of position * inv_freq[i] from the step's table; dimensions from `rot` on pass;
//   then (unit != 0) the head is divided by sqrt(mean(head^2) + eps): a norm without a weight;
//   q goes to q_out; the rotated, normed key goes to the token's slot of k_cache; the first `hdv`
//   values of the key *as projected* (before rotation and norm) go to the slot of v_cache when
//   `v` is null, else the first `hdv` values of the v head.
//
// One warp per (token, head); all arithmetic float32; the inputs may be `nparts` float32 partial
// products [nparts][T][row], added in index order.
#include "common.cuh"

namespace aien {

constexpr int QU_MAX_HEAD = 256;

template <typename TI, typename TC, typename TKV>
__global__ void __launch_bounds__(128)
qk_rope_pairs_unit_kv_write_kernel(
    const TI* __restrict__ q, long q_stride, int nq, const TI* __restrict__ k, long k_stride,
    const TI* __restrict__ v, long v_stride, int nkv, int nparts, size_t part_stride,
    TC* __restrict__ q_out, long q_out_stride, int hd, int hdv, int unit, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
    const int* __restrict__ slot_map, TKV* __restrict__ k_cache, TKV* __restrict__ v_cache) {
    __shared__ float buf[4][QU_MAX_HEAD];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool write_kv = (k != nullptr);
    const int head = blockIdx.y * 4 + warp;
    if (head >= nq + (write_kv ? nkv : 0)) return;
    const bool is_q = head < nq;
    const int hh = is_q ? head : head - nq;
    const long slot = write_kv ? (long)__ldcg(slot_map + t) : -1;
    if (!is_q && slot < 0) return;                                   // the token has no cache slot
    float* hb = buf[warp];
    const TI* src = is_q ? (q + (size_t)t * q_stride + (size_t)hh * hd) : (k + (size_t)t * k_stride + (size_t)hh * hd);
    for (int i = lane; i < hd; i += 32) {
        float val = 0.f;
        for (int p = 0; p < nparts; ++p) val += ld_act(src + (size_t)p * part_stride + i);
        hb[i] = val;
    }
    __syncwarp();
    if (!is_q) {                                                     // the values: the key as projected, or the v head
        TKV* dst = v_cache + ((size_t)slot * nkv + hh) * hdv;
        if (v == nullptr) {
            for (int i = lane; i < hdv; i += 32) dst[i] = from_f<TKV>(hb[i]);
        } else {
            const TI* vs = v + (size_t)t * v_stride + (size_t)hh * hdv;
            for (int i = lane; i < hdv; i += 32) {
                float val = 0.f;
                for (int p = 0; p < nparts; ++p) val += ld_act(vs + (size_t)p * part_stride + i);
                dst[i] = from_f<TKV>(val);
            }
        }
        __syncwarp();
    }
    const int half = rot >> 1;
    if (cos_t != nullptr) {
        for (int i = lane; i < half; i += 32) {
            const float a = hb[2 * i], b = hb[2 * i + 1];
            const float c = __ldcg(cos_t + (size_t)t * half + i), s = __ldcg(sin_t + (size_t)t * half + i);
            hb[2 * i] = a * c - b * s;
            hb[2 * i + 1] = b * c + a * s;
        }
        __syncwarp();
    }
    float scale = 1.0f;
    if (unit) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) ss += hb[i] * hb[i];
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    if (is_q) {
        TC* dst = q_out + (size_t)t * q_out_stride + (size_t)hh * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = from_f<TC>(hb[i] * scale);
    } else {
        TKV* dst = k_cache + ((size_t)slot * nkv + hh) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = from_f<TKV>(hb[i] * scale);
    }
}

// The same with the head in registers: lane l holds the pairs l, l + 32, ... of its head (a pair is one 8- or 4-byte
// load), so the two numbers that turn together sit in one lane, every load of the head and of its cos/sin is issued
// before the first use, and nothing goes through shared memory.  NJ = ceil(hd / 64) pairs a lane.  Needs even strides
// and 8-byte (float32 in) or 4-byte aligned rows; the sums are made in the order of the kernel above per pair, and the
// sum of squares lane by lane and then over the warp: a fixed order of its own, taken for a head size whatever the step.
template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return __ldcg(reinterpret_cast<const float2*>(p)); }
    static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
        const unsigned int r = __ldcg(reinterpret_cast<const unsigned int*>(p));
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    }
};

template <typename TI, typename TC, typename TKV, int NJ>
__global__ void __launch_bounds__(128)
qk_rope_pairs_unit_kv_write_reg_kernel(
    const TI* __restrict__ q, long q_stride, int nq, const TI* __restrict__ k, long k_stride, int nkv, int nparts, size_t part_stride,
    TC* __restrict__ q_out, long q_out_stride, int hd, int hdv, int unit, float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
    const int* __restrict__ slot_map, TKV* __restrict__ k_cache, TKV* __restrict__ v_cache) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool write_kv = (k != nullptr);
    const int head = blockIdx.y * 4 + warp;
    if (head >= nq + (write_kv ? nkv : 0)) return;
    const bool is_q = head < nq;
    const int hh = is_q ? head : head - nq;
    const long slot = write_kv ? (long)__ldcg(slot_map + t) : -1;
    if (!is_q && slot < 0) return;
    const TI* src = is_q ? (q + (size_t)t * q_stride + (size_t)hh * hd) : (k + (size_t)t * k_stride + (size_t)hh * hd);
    const int half = rot >> 1, npairs = hd >> 1;
    float2 v[NJ], cs[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int p = lane + 32 * j;
        v[j] = make_float2(0.f, 0.f);
        cs[j] = make_float2(1.f, 0.f);
        if (p < npairs) {
            for (int part = 0; part < nparts; ++part) {
                const float2 x = Pair<TI>::load(src + (size_t)part * part_stride + 2 * p);
                v[j].x += x.x; v[j].y += x.y;
            }
            if (cos_t != nullptr && p < half) cs[j] = make_float2(__ldcg(cos_t + (size_t)t * half + p), __ldcg(sin_t + (size_t)t * half + p));
        }
    }
    if (!is_q) {                                                     // the values: the key as projected
        TKV* dst = v_cache + ((size_t)slot * nkv + hh) * hdv;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int p = lane + 32 * j;
            if (2 * p + 1 < hdv) Pair<TKV>::store(dst + 2 * p, v[j].x, v[j].y);
            else if (2 * p < hdv) dst[2 * p] = from_f<TKV>(v[j].x);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const float a = v[j].x, b = v[j].y;
        v[j].x = a * cs[j].x - b * cs[j].y;
        v[j].y = b * cs[j].x + a * cs[j].y;
        ss += v[j].x * v[j].x + v[j].y * v[j].y;
    }
    float scale = 1.0f;
    if (unit) scale = 1.0f / sqrtf(warp_sum(ss) / (float)hd + eps);
    if (is_q) {
        TC* dst = q_out + (size_t)t * q_out_stride + (size_t)hh * hd;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int p = lane + 32 * j;
            if (p < npairs) Pair<TC>::store(dst + 2 * p, v[j].x * scale, v[j].y * scale);
        }
    } else {
        TKV* dst = k_cache + ((size_t)slot * nkv + hh) * hd;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int p = lane + 32 * j;
            if (p < npairs) Pair<TKV>::store(dst + 2 * p, v[j].x * scale, v[j].y * scale);
        }
    }
}

}  // namespace aien

using namespace aien;

// in_dt: dtype of q/k/v ([nparts][T][...] float32 when nparts > 1); act_dt: q_out; kv_dt: the caches.
AIEN_API int aien_qk_rope_pairs_unit_kv_write(
    const void* q, long q_stride, int nq, const void* k, long k_stride, const void* v, long v_stride, int nkv,
    int in_dt, int nparts, size_t part_stride, void* q_out, long q_out_stride, int hd, int hdv, int unit, float eps,
    const float* cos_t, const float* sin_t, int rot, const int* slot_map, void* k_cache, void* v_cache,
    int act_dt, int kv_dt, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > QU_MAX_HEAD || hdv <= 0 || hdv > hd || rot < 0 || rot > hd || (rot & 1) || nparts < 1) return AIEN_E_SHAPE;
    if (nparts > 1 && in_dt != AIEN_DT_F32) return AIEN_E_DTYPE;
    const int n_heads = nq + (k != nullptr ? nkv : 0);
    dim3 grid(T, (n_heads + 3) / 4);
    if (grid.y > 65535) return AIEN_E_SHAPE;
    // the head in registers where every row is a whole number of aligned pairs and the values come from the key
    const size_t in_al = in_dt == AIEN_DT_F32 ? 7 : 3, act_al = act_dt == AIEN_DT_F32 ? 7 : 3, kv_al = kv_dt == AIEN_DT_F32 ? 7 : 3;
    const bool pairs_ok = v == nullptr && (hd & 1) == 0 && ((q_stride | k_stride | q_out_stride | (long)part_stride) & 1) == 0 &&
                          (((uintptr_t)q | (uintptr_t)k) & in_al) == 0 && ((uintptr_t)q_out & act_al) == 0 &&
                          (((uintptr_t)k_cache | (uintptr_t)v_cache) & kv_al) == 0 && (hdv & 1) == 0;
    if (pairs_ok) {
        const int nj = (hd + 63) / 64;
#define QU_REG(NJV)                                                                                                          \
        AIEN_DISPATCH_DTYPE(in_dt, TI, AIEN_DISPATCH_DTYPE(act_dt, TC, AIEN_DISPATCH_DTYPE(kv_dt, TKV,                         \
            (launch_chain(qk_rope_pairs_unit_kv_write_reg_kernel<TI, TC, TKV, NJV>, grid, dim3(128), 0, stream,                \
                (const TI*)q, q_stride, nq, (const TI*)k, k_stride, nkv, nparts, part_stride, (TC*)q_out, q_out_stride,        \
                hd, hdv, unit, eps, cos_t, sin_t, rot, slot_map, (TKV*)k_cache, (TKV*)v_cache)))))
        if (nj == 1) { QU_REG(1); } else if (nj == 2) { QU_REG(2); } else if (nj == 3) { QU_REG(3); } else { QU_REG(4); }
#undef QU_REG
        return launch_status();
    }
    AIEN_DISPATCH_DTYPE(in_dt, TI, AIEN_DISPATCH_DTYPE(act_dt, TC, AIEN_DISPATCH_DTYPE(kv_dt, TKV,
        (launch_chain(qk_rope_pairs_unit_kv_write_kernel<TI, TC, TKV>, grid, dim3(128), 0, stream,
            (const TI*)q, q_stride, nq, (const TI*)k, k_stride, (const TI*)v, v_stride, nkv, nparts, part_stride,
            (TC*)q_out, q_out_stride, hd, hdv, unit, eps, cos_t, sin_t, rot, slot_map, (TKV*)k_cache, (TKV*)v_cache)))));
    return launch_status();
}
