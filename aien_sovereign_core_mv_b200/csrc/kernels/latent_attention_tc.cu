// Attention over cached latent rows on the tensor cores (bfloat16 engine): the same result as the plain kernel in
// latent_attention.cu, for latent sizes of 64, 128, 256 or 512 and a rotated part that is a multiple of 16.
//
// A cached row [c | k_rot] serves every head as key and (its first R numbers) as value, so the rows of the score
// product are (token, head) pairs: the queries of a request's portion, laid out [token][head][R + rot], are one
// matrix of len * heads rows.  One CTA owns 64 such rows (16 for steps of single tokens); a step has at most
// T * heads / 64 + S tiles, and a CTA finds its request and offset from q_start.  Keys are visited in blocks of 64 aligned
// to absolute positions, read through the block table into shared memory with cp.async (absent or unneeded rows
// zero-filled).  The warps of a 16-row slab deal out the block's keys for the scores and the latent's channels for the
// weighted sum, so they exchange their row maxima and their probabilities (bfloat16) through shared memory.  Products run
// on mma.sync.m16n8k16 (bfloat16 in, float32
// accumulate) with ldmatrix-fed fragments; masks, the online softmax and the sink are float32 per row.
#include "common.cuh"
#include <math.h>

namespace aien {

constexpr int LX_BM = 64, LX_BN = 64, LX_PSTR = LX_BN + 8;

__device__ __forceinline__ void lx_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void lx_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void lx_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void lx_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lx_ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void lx_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lx_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lx_pack(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// SLABS: 16-row slabs of a tile (4: tiles of 64 rows, for portions; 1: tiles of 16 rows, for steps of single tokens, where
// a request has only its heads as rows).  The WARPS / SLABS warps of a slab deal out the keys of a block for the scores and
// the channels for the weighted sum (tiles of 64 rows run 16 warps: four to a slab, so that a warp's share of the weighted
// sum, 16 rows x a quarter of the latent, leaves registers for loads in flight).
template <int R, int SLABS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, SLABS == 1 ? 2 : 1)
latent_attention_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                           const int* __restrict__ block_table, int max_blocks, const int* __restrict__ q_start,
                           const int* __restrict__ positions, int S, __nv_bfloat16* __restrict__ out,
                           int H, int rd, int page_size, int window, float scale_log2e, const float* __restrict__ sinks,
                           int ksplit, float* __restrict__ part_o, float* __restrict__ part_ml) {
    constexpr int BM = SLABS * 16, PARTS = WARPS / SLABS, KP = LX_BN / PARTS, NJ = KP / 8, CHP = R / PARTS, THREADS = WARPS * 32;
    constexpr int DT = CHP / 8;                  // n8 tiles of this warp's share of the channels
    static_assert(DT >= 2 && DT % 2 == 0, "a warp's share of the latent must be whole pairs of n8 tiles");
    const int D = R + rd, STR = D + 8, CH = D / 8, KS = D / 16;
    extern __shared__ __align__(16) uint8_t lx_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lx_smem);          // [BM][STR]
    __nv_bfloat16* Ks = Qs + BM * STR;                                      // [64][STR]
    __nv_bfloat16* Ps = Ks + LX_BN * STR;                                   // [BM][LX_PSTR]
    float* stat = reinterpret_cast<float*>(Ps + BM * LX_PSTR);              // [PARTS][BM]
    __shared__ int key_there[LX_BN];                                        // whether the block's key is in the cache and needed
    const uint32_t Qs_u = (uint32_t)__cvta_generic_to_shared(Qs), Ks_u = (uint32_t)__cvta_generic_to_shared(Ks);
    const uint32_t Ps_u = (uint32_t)__cvta_generic_to_shared(Ps);

    // which request, which rows
    int s = -1, row0 = 0, acc = 0;
    for (int i = 0; i < S; ++i) {
        const int tiles = ((q_start[i + 1] - q_start[i]) * H + BM - 1) / BM;
        if ((int)blockIdx.x < acc + tiles) {
            s = i;
            row0 = ((int)blockIdx.x - acc) * BM;
            break;
        }
        acc += tiles;
    }
    if (s < 0) return;
    const int qs = q_start[s], len = q_start[s + 1] - qs;
    const int nrows = min(BM, len * H - row0);
    const int pos_first = positions[qs];
    const int pos_lo = pos_first + row0 / H, pos_hi = pos_first + (row0 + nrows - 1) / H;
    const int first = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
    const int* bt = block_table + (size_t)s * max_blocks;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slab = warp % SLABS, half = warp / SLABS;                     // half: which share of the keys / channels
    const int g = lane >> 2, c = lane & 3;

    const __nv_bfloat16* qbase = q + ((size_t)qs * H + row0) * D;
    for (int idx = tid; idx < BM * CH; idx += THREADS) {
        const int r = idx / CH, ch = idx - r * CH;
        const bool valid = r < nrows;
        lx_cp_async16(Qs_u + (uint32_t)(r * STR + ch * 8) * 2, qbase + (size_t)(valid ? r : 0) * D + ch * 8, valid);
    }
    lx_cp_async_commit();

    const uint32_t q_frag_u = Qs_u + (uint32_t)((slab * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * STR + (lane >> 4) * 8) * 2;
    const uint32_t p_frag_u = Ps_u + (uint32_t)((slab * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LX_PSTR + (lane >> 4) * 8) * 2;

    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int ra = slab * 16 + g, rb = ra + 8;                              // this thread's two rows in the tile
    const int qpos0 = ra < nrows ? pos_first + (row0 + ra) / H : -1, qpos1 = rb < nrows ? pos_first + (row0 + rb) / H : -1;
    const int wlo0 = window > 0 ? qpos0 - window + 1 : 0, wlo1 = window > 0 ? qpos1 - window + 1 : 0;
    const bool active = slab * 16 < nrows;

    const int kb_begin = first / LX_BN, kb_end = pos_hi / LX_BN;
    if (ksplit > 1) {                                                      // Q must have landed even if this CTA gets no block
        lx_cp_async_wait_all();
        __syncthreads();
    }
    for (int kb = kb_begin + (int)blockIdx.y; kb <= kb_end; kb += ksplit) {
        for (int idx = tid; idx < LX_BN * CH; idx += THREADS) {
            const int r = idx / CH, ch = idx - r * CH;
            const int key = kb * LX_BN + r;
            bool valid = key >= first && key <= pos_hi;
            long slot = 0;
            if (valid) {
                const int page = bt[key / page_size];
                valid = page >= 0;
                slot = (long)page * page_size + key % page_size;
            }
            lx_cp_async16(Ks_u + (uint32_t)(r * STR + ch * 8) * 2, cache + (size_t)(valid ? slot : 0) * D + ch * 8, valid);
            if (ch == 0) key_there[r] = valid ? 1 : 0;
        }
        lx_cp_async_commit();
        lx_cp_async_wait_all();
        __syncthreads();                                                   // the block's rows (and, first time, Q) have landed

        float sc[NJ][4];
#pragma unroll
        for (int j = 0; j < NJ; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
        if (active) {
#pragma unroll 4
            for (int kk = 0; kk < KS; ++kk) {
                uint32_t q0r, q1r, q2r, q3r;
                lx_ldmatrix_x4(q_frag_u + kk * 32, q0r, q1r, q2r, q3r);
                if constexpr (NJ == 1) {
                    const int row = half * KP + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
                    uint32_t b0, b1;
                    lx_ldmatrix_x2(Ks_u + (uint32_t)(row * STR + col) * 2, b0, b1);
                    lx_mma(sc[0], q0r, q1r, q2r, q3r, b0, b1);
                } else {
#pragma unroll
                    for (int j = 0; j < NJ; j += 2) {
                        const int mi = lane >> 3;
                        const int row = half * KP + (j + (mi >> 1)) * 8 + (lane & 7), col = kk * 16 + (mi & 1) * 8;
                        uint32_t b0, b1, b2, b3;
                        lx_ldmatrix_x4(Ks_u + (uint32_t)(row * STR + col) * 2, b0, b1, b2, b3);
                        lx_mma(sc[j], q0r, q1r, q2r, q3r, b0, b1);
                        lx_mma(sc[j + (NJ > 1 ? 1 : 0)], q0r, q1r, q2r, q3r, b2, b3);
                    }
                }
            }
        }
        // masks and this half's row maxima (scores in log2 units)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kl = half * KP + j * 8 + 2 * c + e, key = kb * LX_BN + kl;
                const bool there = key_there[kl] != 0;
                const bool ok0 = there && key <= qpos0 && key >= wlo0, ok1 = there && key <= qpos1 && key >= wlo1;
                sc[j][e] = ok0 ? sc[j][e] * scale_log2e : -INFINITY;
                sc[j][2 + e] = ok1 ? sc[j][2 + e] * scale_log2e : -INFINITY;
                mx0 = fmaxf(mx0, sc[j][e]);
                mx1 = fmaxf(mx1, sc[j][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (c == 0) {
            stat[half * BM + ra] = mx0;
            stat[half * BM + rb] = mx1;
        }
        __syncthreads();                                                   // every share's maxima are there
#pragma unroll
        for (int pp = 0; pp < PARTS; ++pp) {
            mx0 = fmaxf(mx0, stat[pp * BM + ra]);
            mx1 = fmaxf(mx1, stat[pp * BM + rb]);
        }
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float corr0 = (m_run[0] == -INFINITY) ? 0.f : exp2f(m_run[0] - mn0);
        const float corr1 = (m_run[1] == -INFINITY) ? 0.f : exp2f(m_run[1] - mn1);
        const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            float p00 = exp2f(sc[j][0] - base0), p01 = exp2f(sc[j][1] - base0);      // exp2(-inf) = 0 for masked keys
            float p10 = exp2f(sc[j][2] - base1), p11 = exp2f(sc[j][3] - base1);
            sum0 += p00 + p01;
            sum1 += p10 + p11;
            const int col = half * KP + j * 8 + 2 * c;
            *reinterpret_cast<uint32_t*>(Ps + ra * LX_PSTR + col) = lx_pack(p00, p01);
            *reinterpret_cast<uint32_t*>(Ps + rb * LX_PSTR + col) = lx_pack(p10, p11);
        }
        l_run[0] = l_run[0] * corr0 + sum0;
        l_run[1] = l_run[1] * corr1 + sum1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int d = 0; d < DT; ++d) { o[d][0] *= corr0; o[d][1] *= corr0; o[d][2] *= corr1; o[d][3] *= corr1; }
        __syncthreads();                                                   // the probabilities of every share are there
        if (active) {
#pragma unroll
            for (int ks = 0; ks < LX_BN / 16; ++ks) {
                uint32_t a0, a1, a2, a3;
                lx_ldmatrix_x4(p_frag_u + ks * 32, a0, a1, a2, a3);
#pragma unroll
                for (int d = 0; d < DT; d += 2) {
                    const int row = ks * 16 + (lane & 15), col = half * CHP + (d + (lane >> 4)) * 8;
                    uint32_t b0, b1, b2, b3;
                    lx_ldmatrix_x4_trans(Ks_u + (uint32_t)(row * STR + col) * 2, b0, b1, b2, b3);
                    lx_mma(o[d], a0, a1, a2, a3, b0, b1);
                    lx_mma(o[d + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();                                                   // every warp is done with this block
    }

    if (ksplit > 1) {
        // this CTA saw only some of the key blocks: its running maximum, its sum and its unnormalised weighted sum go to
        // the scratch, and a second launch combines the CTAs of a row
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1); l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1); l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
        if (c == 0) {
            stat[half * BM + ra] = l_run[0];
            stat[half * BM + rb] = l_run[1];
        }
        __syncthreads();
        l_run[0] = l_run[1] = 0.f;
#pragma unroll
        for (int pp = 0; pp < PARTS; ++pp) {
            l_run[0] += stat[pp * BM + ra];
            l_run[1] += stat[pp * BM + rb];
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = r == 0 ? ra : rb;
            if (row >= nrows) continue;
            const size_t slot = ((size_t)qs * H + row0 + row) * ksplit + blockIdx.y;
            if (half == 0 && c == 0) {
                part_ml[slot * 2] = m_run[r];
                part_ml[slot * 2 + 1] = l_run[r];
            }
            float* dst = part_o + slot * R + half * CHP;
#pragma unroll
            for (int d = 0; d < DT; ++d) *reinterpret_cast<float2*>(dst + d * 8 + 2 * c) = make_float2(o[d][2 * r], o[d][2 * r + 1]);
        }
        return;
    }
    // the denominators: this thread's partial sums, its quad's, the other half's
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1); l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1); l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    if (c == 0) {
        stat[half * BM + ra] = l_run[0];
        stat[half * BM + rb] = l_run[1];
    }
    __syncthreads();
    l_run[0] = l_run[1] = 0.f;
#pragma unroll
    for (int pp = 0; pp < PARTS; ++pp) {
        l_run[0] += stat[pp * BM + ra];
        l_run[1] += stat[pp * BM + rb];
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r == 0 ? ra : rb;
        if (row >= nrows) continue;
        float corr = 1.f;
        if (sinks != nullptr) {                                            // the sink joins the denominator once (log2 units like the scores)
            const float sk = sinks[(row0 + row) % H] * 1.4426950408889634f;
            const float mn = fmaxf(m_run[r], sk);
            corr = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - mn);
            l_run[r] = l_run[r] * corr + exp2f(sk - mn);
        }
        const float inv = l_run[r] > 0.f ? corr / l_run[r] : 0.f;
        __nv_bfloat16* dst = out + ((size_t)qs * H + row0 + row) * R + half * CHP;
#pragma unroll
        for (int d = 0; d < DT; ++d)
            *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * c) = lx_pack(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
}

// out[row] = sum_s 2^(m_s - M) o_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)), M = max over the row's parts and the sink
template <int R>
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int ksplit,
                                              const float* __restrict__ sinks, int H, __nv_bfloat16* __restrict__ out) {
    const size_t row = blockIdx.x;
    const float sk = sinks != nullptr ? sinks[row % H] * 1.4426950408889634f : -INFINITY;
    float M = sk;
    for (int s = 0; s < ksplit; ++s) M = fmaxf(M, part_ml[(row * ksplit + s) * 2]);
    float den = (sinks != nullptr && M != -INFINITY) ? exp2f(sk - M) : 0.f;
    for (int s = 0; s < ksplit; ++s) {
        const float m = part_ml[(row * ksplit + s) * 2];
        if (m != -INFINITY) den += exp2f(m - M) * part_ml[(row * ksplit + s) * 2 + 1];
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    for (int ch = threadIdx.x; ch < R; ch += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < ksplit; ++s) {
            const float m = part_ml[(row * ksplit + s) * 2];
            if (m != -INFINITY) acc += exp2f(m - M) * part_o[(row * ksplit + s) * R + ch];
        }
        out[row * R + ch] = __float2bfloat16_rn(acc * inv);
    }
}

template <int R, int SLABS, int WARPS>
static int launch_latent_tc(const void* q, const void* cache, const int* bt, int max_blocks, const int* q_start, const int* positions,
                            int T, int S, void* out, int H, int rd, int page_size, int window, float scale, const float* sinks,
                            int ksplit, float* part_o, float* part_ml, cudaStream_t stream) {
    const int D = R + rd;
    constexpr int BM = SLABS * 16;
    const size_t smem = (size_t)(BM + LX_BN) * (D + 8) * 2 + (size_t)BM * LX_PSTR * 2 + (size_t)WARPS * 16 * sizeof(float);
    if (smem > 227 * 1024) return AIEN_E_SHAPE;
    auto kern = latent_attention_tc_kernel<R, SLABS, WARPS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return AIEN_E_STATE;
    const long tiles = ((long)T * H) / BM + S;
    kern<<<dim3((unsigned)tiles, ksplit), WARPS * 32, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, bt, max_blocks, q_start,
                                                                     positions, S, (__nv_bfloat16*)out, H, rd, page_size, window,
                                                                     scale * 1.4426950408889634f, sinks, ksplit, part_o, part_ml);
    if (ksplit > 1)
        latent_attention_merge_kernel<R><<<dim3((unsigned)((long)T * H)), 128, 0, stream>>>(part_o, part_ml, ksplit, sinks, H, (__nv_bfloat16*)out);
    return launch_status();
}


// ---------------------------------------------------------------- one product per head, on the tensor cores
// C[m, h, n] = sum_k A[m, h, k] * W[h, n, k] (see head_project_kernel) for bfloat16 A and W: tiles of 64 x 64 per CTA of
// four warps, k in steps of 64 through shared memory (cp.async), mma.sync.m16n8k16 with float32 accumulation.
constexpr int HT_BM = 64, HT_BN = 64, HT_BK = 64, HT_STR = HT_BK + 8;

template <typename TC>
__global__ void __launch_bounds__(128)
head_project_tc_kernel(const __nv_bfloat16* __restrict__ A, long lda, long a_head, const __nv_bfloat16* __restrict__ W, long w_head,
                       TC* __restrict__ C, long ldc, long c_head, int M, int N, int K) {
    __shared__ __align__(16) __nv_bfloat16 As[HT_BM * HT_STR];
    __shared__ __align__(16) __nv_bfloat16 Ws[HT_BN * HT_STR];
    const uint32_t As_u = (uint32_t)__cvta_generic_to_shared(As), Ws_u = (uint32_t)__cvta_generic_to_shared(Ws);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mh = warp & 1, nh = warp >> 1, g = lane >> 2, c = lane & 3;
    const int m0 = blockIdx.y * HT_BM, n0 = blockIdx.x * HT_BN, h = blockIdx.z;
    A += (size_t)h * a_head;
    W += (size_t)h * w_head;
    C += (size_t)h * c_head;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HT_BK) {
        for (int idx = tid; idx < HT_BM * (HT_BK / 8); idx += 128) {
            const int r = idx >> 3, ch = idx & 7;
            const bool kin = k0 + ch * 8 < K;
            const bool va = kin && m0 + r < M, vw = kin && n0 + r < N;
            lx_cp_async16(As_u + (uint32_t)(r * HT_STR + ch * 8) * 2, A + (size_t)(va ? m0 + r : 0) * lda + (va ? k0 + ch * 8 : 0), va);
            lx_cp_async16(Ws_u + (uint32_t)(r * HT_STR + ch * 8) * 2, W + (size_t)(vw ? n0 + r : 0) * K + (vw ? k0 + ch * 8 : 0), vw);
        }
        lx_cp_async_commit();
        lx_cp_async_wait_all();
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HT_BK / 16; ++kk) {
            uint32_t a[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
                lx_ldmatrix_x4(As_u + (uint32_t)((mh * 32 + mt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * HT_STR + kk * 16 + (lane >> 4) * 8) * 2,
                               a[mt][0], a[mt][1], a[mt][2], a[mt][3]);
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int mi = lane >> 3;
                uint32_t b0, b1, b2, b3;
                lx_ldmatrix_x4(Ws_u + (uint32_t)((nh * 32 + (j + (mi >> 1)) * 8 + (lane & 7)) * HT_STR + kk * 16 + (mi & 1) * 8) * 2, b0, b1, b2, b3);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    lx_mma(acc[mt][j], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
                    lx_mma(acc[mt][j + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = m0 + mh * 32 + mt * 16 + g + (e >> 1) * 8, n = n0 + nh * 32 + j * 8 + 2 * c + (e & 1);
                if (m < M && n < N) C[(size_t)m * ldc + n] = from_f<TC>(acc[mt][j][e]);
            }
}

}  // namespace aien

using namespace aien;

AIEN_API int aien_latent_attention_tc_supports(int kv_rank, int rot_dim) {
    if (!(kv_rank == 64 || kv_rank == 128 || kv_rank == 256 || kv_rank == 512) || rot_dim < 0 || (rot_dim & 15)) return 0;
    const size_t smem = (size_t)(LX_BM + LX_BN) * (kv_rank + rot_dim + 8) * 2 + (size_t)LX_BM * LX_PSTR * 2 + 16 * 16 * sizeof(float);
    return smem <= 227 * 1024 ? 1 : 0;
}

// q bfloat16 [T, H, kv_rank + rot_dim] (contiguous), cache bfloat16 [slots, kv_rank + rot_dim], out bfloat16 [T, H, kv_rank].
// The step's T tokens are the portions q_start[s] .. q_start[s + 1] of S requests; positions[t] is token t's position.
// ksplit > 1: the key blocks of every tile are dealt out to ksplit CTAs (for steps with few tiles); part_o (float32,
// T * H * ksplit * kv_rank) and part_ml (float32, T * H * ksplit * 2) hold their partial results for the merging launch.
// small_tiles != 0: tiles of 16 rows instead of 64 (steps in which every request brings one token), for latents of 128 and more.
AIEN_API int aien_latent_attention_tc(const void* q, const void* cache, const int* block_table, int max_blocks, const int* q_start,
                                      const int* positions, void* out, int T, int S, int H, int kv_rank, int rot_dim, int page_size,
                                      int window, float scale, const float* sinks, int ksplit, float* part_o, float* part_ml,
                                      int small_tiles, cudaStream_t stream) {
    if (T <= 0 || S <= 0) return 0;
    if (H <= 0 || page_size <= 0 || window < 0 || !aien_latent_attention_tc_supports(kv_rank, rot_dim)) return AIEN_E_SHAPE;
    if (((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 3)) return AIEN_E_ALIGN;
    if (ksplit < 1 || ksplit > 65535 || (ksplit > 1 && (part_o == nullptr || part_ml == nullptr || ((uintptr_t)part_o & 7)))) return AIEN_E_SHAPE;
#define LX_CASE(RV, SL)                                                                                                          \
    if (kv_rank == RV)                                                                                                           \
        return launch_latent_tc<RV, SL, (SL == 4 ? 16 : 8)>(q, cache, block_table, max_blocks, q_start, positions, T, S, out, H, rot_dim, page_size,  \
                                        window, scale, sinks, ksplit, part_o, part_ml, stream);
    if (small_tiles && kv_rank >= 128) {                   // tiles of 16 rows: a latent of 64 would leave a warp half a pair of n8 tiles
        LX_CASE(128, 1) LX_CASE(256, 1) LX_CASE(512, 1)
    }
    LX_CASE(64, 4) LX_CASE(128, 4) LX_CASE(256, 4) LX_CASE(512, 4)
#undef LX_CASE
    return AIEN_E_SHAPE;
}

// A bfloat16 [M, lda] (head h at column h * a_head), W bfloat16 [heads, N, K], C [M, ldc] (head h at column h * c_head).
// K, lda and a_head multiples of 8, A and W 16-byte aligned.
AIEN_API int aien_head_project_tc(const void* A, long lda, long a_head, const void* W, void* C, int c_dt, long ldc, long c_head,
                                  int M, int N, int K, int heads, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return 0;
    if (K <= 0 || heads > 65535) return AIEN_E_SHAPE;
    if ((K & 7) || (lda & 7) || (a_head & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return AIEN_E_ALIGN;
    dim3 grid((N + HT_BN - 1) / HT_BN, (M + HT_BM - 1) / HT_BM, heads);
    if (grid.y > 65535) return AIEN_E_SHAPE;
    AIEN_DISPATCH_DTYPE(c_dt, TC, (head_project_tc_kernel<TC><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)A, lda, a_head, (const __nv_bfloat16*)W,
                                                                                     (long)N * K, (TC*)C, ldc, c_head, M, N, K)));
    return launch_status();
}
