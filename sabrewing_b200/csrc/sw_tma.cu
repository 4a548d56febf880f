// TMA-staged grouped int4 expert products (decode-size groups).
//
// Same arithmetic as sw_mma.cu (subnormal-nibble A fragments, fp16 hi/lo packed
// activations, per-step tensor-core partial sums, "-8 * sum x" correction), but
// no thread issues a global load: one producer warp per CTA streams
//   - the weight rows of the CTA's work item as 2D TMA tiles
//     (cp.async.bulk.tensor, 128-byte rows = 256 columns per stage, 128B swizzle)
//   - the packed activation rows of the group as 1-KB bulk copies
// into a ring of shared-memory stages guarded by full/empty mbarriers, and four
// consumer warps read their fragments from shared memory.  The activation tile
// of a stage is shared by all consumer warps of the CTA.
//
// CTA work item = (group, block of 4 warps x MT m-tiles): gate/up = 32*MT
// (gate,up) row pairs, down = 64*MT rows.  Row g of an m-tile lives at tile row
// rho(g) = (g>>1)|((g&1)<<2) so that the two row groups of a quarter-warp differ
// in swizzle bit 2 and all 16-byte fragment reads are bank-conflict free.
//
// Every mbarrier wait is bounded; a wait that runs out sets SW_ST_TIMEOUT in the
// status word, raises a CTA-wide abort flag and every thread leaves its loops.
#include "sw_common.cuh"
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#define SW_TMA_STAGE_COLS 256
#define SW_TMA_BROW (1024 + 16)          // bytes per activation row of a stage (padded against bank conflicts)
#define SW_WAIT_LIMIT (1u << 24)

__device__ __forceinline__ unsigned sw_smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sw_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void sw_mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sw_mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool sw_mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag, unsigned limit = SW_WAIT_LIMIT) {
    for (unsigned it = 0; it < limit; it++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void sw_tma_load_2d(unsigned dst, const CUtensorMap *tm, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void sw_bulk_load(unsigned dst, const void *src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void sw_mma_f16_t(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sw_dq4_t(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t w2 = w >> 8;
    h[0] = w & 0x000F000Fu; h[1] = w & 0x00F000F0u; h[2] = w2 & 0x000F000Fu; h[3] = w2 & 0x00F000F0u;
}
__device__ __forceinline__ uint32_t sw_word_t(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ size_t sw_packed_pos_t(int col) {
    const int c8 = col >> 3, s = c8 >> 4, tt = (c8 >> 2) & 3, wi = c8 & 3, j = col & 7;
    return (size_t)(((s * 4 + wi) * 4 + tt) * 16 + ((j & 3) * 2 + (j >> 2)));
}
__device__ __forceinline__ float sw_split_f16_t(float v, __half &hi, __half &lo) {
    v = fminf(fmaxf(v, -65504.f), 65504.f);
    hi = __float2half_rn(v);
    const float h = __half2float(hi);
    lo = __float2half_rn(v - h);
    return h + __half2float(lo);
}
#define SW_ACC_SCALE_T 16777216.f

struct SwTmaArgs {
    const float *Ws;
    const unsigned char *XP;       // packed activation rows (bytes)
    const float *xsum; int xsum_parts;
    void *Yout; float *ypart;
    const int *gexp, *gbeg, *gcnt, *Gp, *grow;
    int *status;
    int KD, OUT, expert_lo, expert_cnt;
    const float *rex;              // per-row powers of two (null = 1): gate/up by token row, down by packed row
    float *srex_out;               // gate/up: the token's power of two, copied per packed row for the down product
};

// fragments of one stage (two 128-column steps) from shared memory -> MT m-tiles of accumulators
template <bool GATEUP, int MT, bool M8>
__device__ __forceinline__ void sw_tma_stage(float (&acc)[MT][4], const unsigned char *sp, int warp, int rho, int t, int bofs) {
    constexpr int ABYTES = 64 * MT * 128;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        float part[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) part[mt][i] = 0.f;
        uint4 wa[MT], wb[MT];
        const int chunk = ((j * 4 + t) ^ rho) * 16;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            if (GATEUP) {
                const int tr = warp * (8 * MT) + mt * 8 + rho;
                wa[mt] = *reinterpret_cast<const uint4 *>(sp + tr * 128 + chunk);
                wb[mt] = *reinterpret_cast<const uint4 *>(sp + ABYTES / 2 + tr * 128 + chunk);
            } else {
                const int tr = warp * (16 * MT) + mt * 16 + rho;
                wa[mt] = *reinterpret_cast<const uint4 *>(sp + tr * 128 + chunk);
                wb[mt] = *reinterpret_cast<const uint4 *>(sp + (tr + 8) * 128 + chunk);
            }
        }
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            const uint4 b0 = *reinterpret_cast<const uint4 *>(sp + bofs + (j * 4 + wi) * 128);
            uint4 b1;
            if (M8) b1 = *reinterpret_cast<const uint4 *>(sp + bofs + (j * 4 + wi) * 128 + 16);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                uint32_t ga[4], ua[4];
                sw_dq4_t(sw_word_t(wa[mt], wi), ga);
                sw_dq4_t(sw_word_t(wb[mt], wi), ua);
                sw_mma_f16_t(part[mt], ga[0], ua[0], ga[1], ua[1], b0.x, b0.y);
                sw_mma_f16_t(part[mt], ga[2], ua[2], ga[3], ua[3], b0.z, b0.w);
                if (M8) {
                    sw_mma_f16_t(part[mt], ga[0], ua[0], ga[1], ua[1], b1.x, b1.y);
                    sw_mma_f16_t(part[mt], ga[2], ua[2], ga[3], ua[3], b1.z, b1.w);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[mt][i] += part[mt][i];
    }
}

// Shared-memory stage: [A tile(s): 128 rows x 128 B, 1024-aligned][B: 8 rows x SW_TMA_BROW]
template <bool GATEUP, int MT, int P>
__global__ void __launch_bounds__(160)
k_q4_tma(const __grid_constant__ CUtensorMap tmW, const SwTmaArgs a) {
    constexpr int AROWS = 64 * MT;                 // weight rows per stage (gate/up: 32*MT gate + 32*MT up)
    constexpr int ABYTES = AROWS * 128;
    constexpr int BBYTES = 8 * SW_TMA_BROW;
    constexpr int STAGE_BYTES = ((ABYTES + BBYTES + 1023) / 1024) * 1024;
    constexpr int OPI = GATEUP ? 32 * MT : 64 * MT;   // outputs per CTA item
    extern __shared__ unsigned char sw_dyn[];
    __shared__ unsigned long long s_full[P], s_empty[P];
    __shared__ int s_abort;
    // 8 * (row sum of the token's activations) for the up to 8 token rows of a pass, written by the producer warp
    // (ring of 8 passes: the producer is at most P <= 6 passes ahead of the consumers' epilogue)
    __shared__ float s_corr[8][8];
    __shared__ float s_rex[8][8];                  // the rows' powers of two, same ring
    unsigned char *smem = (unsigned char *)(((uintptr_t)sw_dyn + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KD = a.KD, OUT = a.OUT;
    const int nrows_w = GATEUP ? 2 * OUT : OUT;
    const int NST = (KD + SW_TMA_STAGE_COLS - 1) / SW_TMA_STAGE_COLS;   // stages per pass
    const int G = *a.Gp;
    const int rb_per_group = (OUT + OPI - 1) / OPI;
    const int items = G * rb_per_group;
    const size_t xrow_bytes = (size_t)KD * 4;

    if (threadIdx.x == 0) {
        for (int i = 0; i < P; i++) { sw_mbar_init(sw_smem_u32(&s_full[i]), 1); sw_mbar_init(sw_smem_u32(&s_empty[i]), 4); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // activation tiles start from zeros: a short last stage multiplies stale bytes by zero weights only
    for (int i = threadIdx.x; i < P * (BBYTES / 16); i += blockDim.x) {
        const int st = i / (BBYTES / 16), o = i - st * (BBYTES / 16);
        reinterpret_cast<uint4 *>(smem + (size_t)st * STAGE_BYTES + ABYTES)[o] = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    volatile int *abortp = &s_abort;

    if (warp == 4) {
        // ------------------------------ producer ------------------------------
        // Lane 0 streams the stages.  All lanes together also fetch the row-sum partials of the pass's token rows
        // (the epilogue needs 8 * sum(x) per token row to undo the +8 of the unsigned nibbles), add them in a fixed
        // order and leave the results in s_corr before the pass's LAST stage is announced: the consumers, who wait
        // for that stage before their epilogue, then find them without touching global memory.
        unsigned it = 0, pass = 0;                      // global stage and pass counters of this CTA
        for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x) {
            const int gi = item / rb_per_group, rb = item - gi * rb_per_group;
            const int e = a.gexp[gi] - a.expert_lo;
            if (e < 0 || e >= a.expert_cnt) continue;
            const int n = a.gcnt[gi], beg = a.gbeg[gi];
            const int row0 = e * nrows_w + rb * OPI;
            for (int c0 = 0; c0 < n && !*abortp; pass++) {
                const bool m8 = n - c0 > 4;
                const int ntok = m8 ? min(8, n - c0) : n - c0;
                // partial sums of row r: lane l takes parts l, l+32, ... (ascending); eight rows' loads are in flight at once
                float v[8];
#pragma unroll
                for (int r = 0; r < 8; r++) v[r] = 0.f;
                float my_rex = 1.f;                                                // lane r: the power of two of row r
                if (lane < ntok && a.rex) my_rex = a.rex[GATEUP ? a.grow[beg + c0 + lane] : beg + c0 + lane];   // used at the join below
                for (int k = lane; k < a.xsum_parts; k += 32) {
                    float ld[8];
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        ld[r] = 0.f;
                        if (r < ntok) {
                            const int rid = GATEUP ? a.grow[beg + c0 + r] : beg + c0 + r;
                            ld[r] = a.xsum[(size_t)rid * a.xsum_parts + k];
                        }
                    }
#pragma unroll
                    for (int r = 0; r < 8; r++) v[r] += ld[r];
                }
                bool dead = false;
                for (int st = 0; st < NST; st++, it++) {
                    if (st == NST - 1) {
                        // join: reduce over the lanes in a fixed tree, publish, then announce the last stage
#pragma unroll
                        for (int r = 0; r < 8; r++) {
                            float sx = v[r];
#pragma unroll
                            for (int off = 16; off; off >>= 1) sx += __shfl_xor_sync(SW_FULL_MASK, sx, off);
                            if (lane == 0) s_corr[pass & 7][r] = 8.f * sx;
                        }
                        if (lane < 8) s_rex[pass & 7][lane] = my_rex;
                        if (GATEUP && a.srex_out && rb == 0 && lane < ntok) a.srex_out[beg + c0 + lane] = my_rex;
                        __syncwarp();
                    }
                    if (lane == 0) {
                        const int slot = it % P;
                        if (it >= (unsigned)P && !sw_mbar_wait(sw_smem_u32(&s_empty[slot]), ((it / P) - 1) & 1, abortp)) {
                            atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; dead = true;
                        } else {
                            unsigned char *sp = smem + (size_t)slot * STAGE_BYTES;
                            const unsigned bar = sw_smem_u32(&s_full[slot]);
                            const int colb = st * 128;                                  // byte column of the stage
                            const int bcols = min(SW_TMA_STAGE_COLS, KD - st * SW_TMA_STAGE_COLS);
                            const unsigned bbytes = (unsigned)bcols * 4;
                            sw_mbar_expect_tx(bar, (unsigned)ABYTES + (unsigned)ntok * bbytes);
                            if (GATEUP) {
                                sw_tma_load_2d(sw_smem_u32(sp), &tmW, colb, row0, bar);
                                sw_tma_load_2d(sw_smem_u32(sp + ABYTES / 2), &tmW, colb, row0 + OUT, bar);
                            } else {
                                sw_tma_load_2d(sw_smem_u32(sp), &tmW, colb, row0, bar);
                                if (MT == 4) sw_tma_load_2d(sw_smem_u32(sp + ABYTES / 2), &tmW, colb, row0 + AROWS / 2, bar);
                            }
                            for (int r = 0; r < ntok; r++) {
                                const int rowid = GATEUP ? a.grow[beg + c0 + r] : beg + c0 + r;
                                sw_bulk_load(sw_smem_u32(sp + ABYTES + r * SW_TMA_BROW),
                                             a.XP + (size_t)rowid * xrow_bytes + (size_t)st * (SW_TMA_STAGE_COLS * 4), bbytes, bar);
                            }
                        }
                    }
                    dead = __shfl_sync(SW_FULL_MASK, dead, 0);
                    if (dead) break;
                }
                if (dead) break;
                c0 += ntok;
            }
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int g = lane >> 2, t = lane & 3;
        const int rho = (g >> 1) | ((g & 1) << 2);
        unsigned it = 0, pass = 0;
        bool clamped = false;                                             // a SiLU*up value left the fp16 range
        // group of the next item, fetched one item ahead (its L2 round trip then passes under the current item)
        int nx_e = 0, nx_n = 0, nx_beg = 0;
        if ((int)blockIdx.x < items) { const int g0 = blockIdx.x / rb_per_group; nx_e = a.gexp[g0]; nx_n = a.gcnt[g0]; nx_beg = a.gbeg[g0]; }
        for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x) {
            const int gi = item / rb_per_group, rb = item - gi * rb_per_group;
            const int e = nx_e - a.expert_lo, n = nx_n, beg = nx_beg;
            if (item + (int)gridDim.x < items) {
                const int g1 = (item + gridDim.x) / rb_per_group;
                nx_e = a.gexp[g1]; nx_n = a.gcnt[g1]; nx_beg = a.gbeg[g1];
            }
            if (e < 0 || e >= a.expert_cnt) continue;
            const float *ws = a.Ws + (size_t)e * nrows_w;
            // the scales of this thread's rows, requested before the K loop so that the epilogue does not wait for them
            float sc0[MT], sc1[MT];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                if (GATEUP) {
                    const int o = rb * OPI + warp * (8 * MT) + mt * 8 + rho;
                    sc0[mt] = o < OUT ? ws[o] : 0.f; sc1[mt] = o < OUT ? ws[OUT + o] : 0.f;
                } else {
                    const int oa = rb * OPI + warp * (16 * MT) + mt * 16 + rho, ob = oa + 8;
                    sc0[mt] = oa < OUT ? ws[oa] : 0.f; sc1[mt] = ob < OUT ? ws[ob] : 0.f;
                }
            }
            // tile rows of this thread: role "row g" and role "row g+8" of m-tile mt
            // gate/up: A tile = [32*MT gate rows][32*MT up rows]; down: [64*MT rows]
            for (int c0 = 0; c0 < n && !*abortp; pass++) {
                const bool m8 = n - c0 > 4;
                const int ntok = m8 ? min(8, n - c0) : n - c0;
                const int brow = m8 ? min(g, ntok - 1) : min(g & 3, ntok - 1);
                const int bofs = ABYTES + brow * SW_TMA_BROW + t * 32 + ((!m8 && g >= 4) ? 16 : 0);
                float acc[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[mt][i] = 0.f;

                for (int st = 0; st < NST; st++, it++) {
                    const int slot = it % P;
                    if (!sw_mbar_wait(sw_smem_u32(&s_full[slot]), (it / P) & 1, abortp)) {
                        if (lane == 0) { atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; }
                        break;
                    }
                    const unsigned char *sp = smem + (size_t)slot * STAGE_BYTES;
                    if (m8) sw_tma_stage<GATEUP, MT, true>(acc, sp, warp, rho, t, bofs);
                    else    sw_tma_stage<GATEUP, MT, false>(acc, sp, warp, rho, t, bofs);
                    __syncwarp();
                    if (lane == 0) sw_mbar_arrive(sw_smem_u32(&s_empty[slot]));
                }
                if (*abortp) break;

                // ---- epilogue (same as the cp.async kernel, rows through rho) ----
                if (!m8) {
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[mt][i] += __shfl_down_sync(SW_FULL_MASK, acc[mt][i], 2);
                }
                const bool own = m8 || t < 2;
                float corr[2], rex[2], rex2[2]; int tok[2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    tok[j] = c0 + 2 * t + j;
                    const bool ok = own && tok[j] < c0 + ntok;
                    corr[j] = ok ? s_corr[pass & 7][2 * t + j] : 0.f;     // left there by the producer warp
                    rex[j] = ok ? s_rex[pass & 7][2 * t + j] : 1.f;
                    rex2[j] = GATEUP ? __frcp_rn(rex[j]) : rex[j] * rex[j];   // gate/up: 2^-e; down: 2^2e (SiLU(gate)*up came in divided by it)
                    if (!ok) tok[j] = -1;
                }
                if (GATEUP) {
                    __half *Y = reinterpret_cast<__half *>(a.Yout);
                    float ysum[2] = {0.f, 0.f};
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        const int o = rb * OPI + warp * (8 * MT) + mt * 8 + rho;
                        const bool ov = o < OUT;
                        const float sg = sc0[mt], su = sc1[mt];
                        const size_t pos = sw_packed_pos_t(ov ? o : 0);
                        const float pre = (o & 1) ? 0.0625f : 1.f;
#pragma unroll
                        for (int j = 0; j < 2; j++) {
                            if (tok[j] < 0 || !ov) continue;
                            // gate at its true size; the up value stays divided by 2^e and the product is divided once more
                            const float gv = (acc[mt][j] * SW_ACC_SCALE_T - corr[j]) * sg * rex[j];
                            const float uv = (acc[mt][2 + j] * SW_ACC_SCALE_T - corr[j]) * su;
                            const float y = ((gv / (1.f + expf(-gv))) * rex2[j]) * uv;
                            __half hi, lo;
                            clamped |= fabsf(y * pre) > 65504.f;
                            const float rep = sw_split_f16_t(y * pre, hi, lo);
                            ysum[j] += (o & 1) ? rep * 16.f : rep;
                            __half *row = Y + (size_t)(beg + tok[j]) * (2 * (size_t)OUT);
                            row[pos] = hi; row[pos + 8] = lo;
                        }
                    }
                    // per packed row: one partial sum per (CTA item, warp), added in order by the down product
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float v = ysum[j];
                        v += __shfl_xor_sync(SW_FULL_MASK, v, 4);
                        v += __shfl_xor_sync(SW_FULL_MASK, v, 8);
                        v += __shfl_xor_sync(SW_FULL_MASK, v, 16);
                        if (g == 0 && tok[j] >= 0) a.ypart[(size_t)(beg + tok[j]) * (rb_per_group * 4) + rb * 4 + warp] = v;
                    }
                } else {
                    float *Y = reinterpret_cast<float *>(a.Yout);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        const int oa = rb * OPI + warp * (16 * MT) + mt * 16 + rho, ob = oa + 8;
                        const float sa = sc0[mt], sb = sc1[mt];
#pragma unroll
                        for (int j = 0; j < 2; j++) {
                            if (tok[j] < 0) continue;
                            float *row = Y + (size_t)(beg + tok[j]) * OUT;
                            if (oa < OUT) row[oa] = (acc[mt][j] * SW_ACC_SCALE_T - corr[j]) * sa * rex2[j];
                            if (ob < OUT) row[ob] = (acc[mt][2 + j] * SW_ACC_SCALE_T - corr[j]) * sb * rex2[j];
                        }
                    }
                }
                c0 += ntok;
            }
        }
        if (GATEUP && clamped) atomicOr(a.status, SW_ST_RANGE);
    }
}

// A wait that must run out: one CTA waits `limit` iterations on a barrier nobody arrives at, then reports through the
// status word exactly as the expert kernels do (SW_ST_TIMEOUT, clean return).  Exercises the give-up path of
// sw_mbar_wait without faulting or hanging anything.
__global__ void k_wait_runs_out(int *status, unsigned limit) {
    __shared__ unsigned long long bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        sw_mbar_init(sw_smem_u32(&bar), 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0 && !sw_mbar_wait(sw_smem_u32(&bar), 0, &s_abort, limit)) atomicOr(status, SW_ST_TIMEOUT);
}
int sw_launch_wait_runs_out(const SwLaunchCfg &c, int *status, unsigned limit) {
    k_wait_runs_out<<<1, 32, 0, c.stream>>>(status, limit);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// Host side: tensor maps (cached per weight blob) and launch.
// ---------------------------------------------------------------------------
typedef CUresult (*sw_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static sw_encode_fn sw_get_encode() {
    // looked up once (thread-safe static initialisation); NULL when the driver does not export the encoder
    static const sw_encode_fn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            return (sw_encode_fn)p;
        cudaGetLastError();
        return (sw_encode_fn)nullptr;
    }();
    return fn;
}

// Cache of encoded tensor maps, keyed by (device, blob pointer, row bytes, rows, box rows).  Guarded by a mutex
// and handed out BY VALUE: an entry may be recycled by another thread while a launch still uses its copy.
struct SwMapKey { int dev; const void *ptr; int rowbytes, boxrows; long long rows; };
struct SwMapEntry { SwMapKey k; CUtensorMap m; };
static SwMapEntry g_maps[64];
static int g_nmaps = 0, g_map_next = 0;
static std::mutex g_maps_mu;

static bool sw_key_eq(const SwMapKey &a, const SwMapKey &b) {
    return a.dev == b.dev && a.ptr == b.ptr && a.rowbytes == b.rowbytes && a.boxrows == b.boxrows && a.rows == b.rows;
}

// enc: the driver's cuTensorMapEncodeTiled (or a stand-in of the host self-test)
static int sw_get_map_with(sw_encode_fn enc, int dev, const void *ptr, int rowbytes, long long rows, int boxrows, CUtensorMap *out) {
    const SwMapKey key{dev, ptr, rowbytes, boxrows, rows};
    std::lock_guard<std::mutex> g(g_maps_mu);
    for (int i = 0; i < g_nmaps; i++)
        if (sw_key_eq(g_maps[i].k, key)) { *out = g_maps[i].m; return 0; }
    if (!enc) return -1;
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)rowbytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)rowbytes};
    cuuint32_t box[2] = {128, (cuuint32_t)boxrows};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return -1;
    const int slot = g_nmaps < 64 ? g_nmaps++ : (g_map_next++ % 64);
    g_maps[slot].k = key; g_maps[slot].m = m;
    *out = m;
    return 0;
}

// Host-only check of the cache keying (no device needed): a stand-in encoder counts its calls and stamps the map
// with them.  Returns 0 when every lookup behaved, else the number of the failed check.
static int g_fake_calls = 0;
static CUresult sw_fake_encode(CUtensorMap *m, CUtensorMapDataType, cuuint32_t, void *ptr, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
    memset(m, 0, sizeof *m); g_fake_calls++;
    memcpy(m, &g_fake_calls, sizeof g_fake_calls); memcpy((char *)m + 8, &ptr, sizeof ptr);
    return CUDA_SUCCESS;
}
int sw_selftest_map_cache() {
    { std::lock_guard<std::mutex> g(g_maps_mu); g_nmaps = 0; g_map_next = 0; }
    g_fake_calls = 0;
    CUtensorMap a, b, c2;
    char blob[4];
    if (sw_get_map_with(sw_fake_encode, 0, blob, 2048, 100, 64, &a) || g_fake_calls != 1) return 1;
    if (sw_get_map_with(sw_fake_encode, 0, blob, 2048, 100, 64, &b) || g_fake_calls != 1 || memcmp(&a, &b, sizeof a)) return 2;   // hit
    if (sw_get_map_with(sw_fake_encode, 1, blob, 2048, 100, 64, &c2) || g_fake_calls != 2) return 3;                              // other device: miss
    if (sw_get_map_with(sw_fake_encode, 0, blob, 2048, 100, 128, &c2) || g_fake_calls != 3) return 4;                             // other box: miss
    if (sw_get_map_with(sw_fake_encode, 0, blob + 1, 2048, 100, 64, &c2) || g_fake_calls != 4) return 5;                         // other blob: miss
    for (int i = 0; i < 80; i++) if (sw_get_map_with(sw_fake_encode, 2, blob, 2048, 1000 + i, 64, &c2)) return 6;                 // more entries than slots: recycled
    if (sw_get_map_with(sw_fake_encode, 2, blob, 2048, 1079, 64, &b) || g_fake_calls != 84) return 7;                             // the newest is still there
    if (sw_get_map_with(nullptr, 3, blob, 2048, 1, 64, &b) == 0) return 8;                                                        // no encoder: a miss fails
    { std::lock_guard<std::mutex> g(g_maps_mu); g_nmaps = 0; g_map_next = 0; }
    return 0;
}

template <bool GATEUP, int MT, int P>
static int sw_launch_q4_tma_t(const SwLaunchCfg &c, const SwQ4Args &a, const SwMmaIO &io, int *status, long long rows_total) {
    constexpr int AROWS = 64 * MT;
    constexpr int STAGE_BYTES = ((AROWS * 128 + 8 * SW_TMA_BROW + 1023) / 1024) * 1024;
    constexpr int SMEM = P * STAGE_BYTES + 1024;
    constexpr int OPI = GATEUP ? 32 * MT : 64 * MT;
    constexpr int BOXROWS = GATEUP ? 32 * MT : (MT == 4 ? 128 : 64 * MT);
    static SwPerDevice per_dev;                       // resident CTAs per SM of this instantiation, per device
    auto kern = k_q4_tma<GATEUP, MT, P>;
    const int ctas_per_sm = per_dev.get(c.dev, [&] {
        int n = 0;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 160, SMEM) != cudaSuccess || n < 1) { cudaGetLastError(); n = 1; }
        return n; });
    if (ctas_per_sm <= 0) return -1;
    CUtensorMap tm;
    if (sw_get_map_with(sw_get_encode(), c.dev, a.q, a.KD / 2, rows_total, BOXROWS, &tm)) return -1;
    SwTmaArgs ka;
    ka.Ws = a.s; ka.XP = (const unsigned char *)io.XP; ka.xsum = io.xsum; ka.xsum_parts = io.xsum_parts;
    ka.Yout = io.Y; ka.ypart = io.ypart; ka.gexp = a.gexp; ka.gbeg = a.gbeg; ka.gcnt = a.gcnt; ka.Gp = a.G; ka.grow = a.grow;
    ka.status = status; ka.KD = a.KD; ka.OUT = a.OUT; ka.expert_lo = a.expert_lo; ka.expert_cnt = a.expert_cnt;
    ka.rex = io.rex; ka.srex_out = io.srex_out;
    long long items = (long long)a.max_groups * ((a.OUT + OPI - 1) / OPI);
    long long grid = (long long)c.num_sms * ctas_per_sm;
    if (grid > items) grid = items;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, 160, SMEM, c.stream>>>(tm, ka);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ypart slots per packed row written by the gate/up launch for a given MT
int sw_q4_tma_parts(int OUT, int mt) { return ((OUT + 32 * mt - 1) / (32 * mt)) * 4; }

bool sw_tma_available() { return sw_get_encode() != nullptr; }

// rows_total: rows of the weight blob visible through a.q (bounds the tensor map; rows past it read as zero)
int sw_launch_q4_tma(const SwLaunchCfg &c, const SwQ4Args &a, const SwMmaIO &io, int *status, long long rows_total, bool gateup, int mt) {
    if (a.max_groups <= 0 || a.max_rows <= 0) return 0;
    if (a.KD % 128 || a.OUT <= 0 || ((uintptr_t)a.q & 15)) return -1;
    const int p_env = sw_tuning().tma_p;     // SW_TMA_P=2|3|4|6: ring depth (tuning knob)
    const int P = p_env ? p_env : 2;          // shallow rings, more resident CTAs: measured best on B200
#define SW_TMA_CASE(G, M, PP) if (mt == M && P == PP) return sw_launch_q4_tma_t<G, M, PP>(c, a, io, status, rows_total)
    if (gateup) {
        SW_TMA_CASE(true, 2, 2); SW_TMA_CASE(true, 2, 3); SW_TMA_CASE(true, 2, 4);
        SW_TMA_CASE(true, 1, 2); SW_TMA_CASE(true, 1, 3); SW_TMA_CASE(true, 1, 4); SW_TMA_CASE(true, 1, 6);
    } else {
        SW_TMA_CASE(false, 2, 2); SW_TMA_CASE(false, 2, 3); SW_TMA_CASE(false, 2, 4);
        SW_TMA_CASE(false, 1, 2); SW_TMA_CASE(false, 1, 3); SW_TMA_CASE(false, 1, 4); SW_TMA_CASE(false, 1, 6);
    }
#undef SW_TMA_CASE
    return -1;
}
