// Bandwidth-bound grouped int4 expert products for decode-size groups.
//
// Every warp streams whole weight rows (16-byte cp.async copies into a private
// shared-memory ring), dequantises the nibbles in registers straight into
// tensor-core A fragments and multiplies them with activation B fragments that
// were pre-split into fp16 hi + lo halves (x = hi + lo to ~21 bits),
// accumulating in f32.  The per-row f32 scale is applied in the epilogue as
// acc*scale[o], like the reference (c/moe_quant.h:104,
// c/backend_cuda_laguna.cu:156).  No CTA-wide synchronisation: a warp is the
// unit of work.
//
// Dequantisation without arithmetic.  A nibble n masked in place into the low
// mantissa bits of an fp16 is the subnormal n*2^-24 (bits 0..3) or n*2^-20 (bits
// 4..7); both are exact tensor-core operands.  So the A fragments are just
// (w & 0x000F000F), (w & 0x00F000F0) of the weight word and of the word shifted
// by 8: five integer instructions per eight weights.  The factor 16 of the
// odd columns is taken out of the activations when they are packed (x/16 there),
// and the "-8" of value = nibble-8 is restored in the epilogue:
//     dot = 2^24 * acc - 8 * sum_k x_k
// with the row sums of the activations computed once where the rows are produced.
//
// Fragment bookkeeping (m16n8k16, lane = 4*g + t):
//   A rows g / g+8 are two weight rows; for gate/up they are gate row i and up
//   row I+i, so the SiLU(gate)*up epilogue is thread-local.
//   A thread's 16 bytes of a weight row are 32 consecutive columns; one 32-bit
//   word (8 columns c0..c7) gives the half2 pairs (c0,c4)(c1,c5)(c2,c6)(c3,c7),
//   which feed two MMAs as k-slots {2t,2t+1 | 2t+8,2t+9}.  The activations are
//   stored in exactly that order ("packed rows"), so the B fragments of those two
//   MMAs are one 16-byte load.
//   B columns: groups of up to 4 token rows put the hi halves of tokens 0..3 in
//   columns 0..3 and their lo halves in columns 4..7 (one MMA per tile, the two
//   column halves are added in the epilogue); groups of 5..8 rows use one MMA for
//   hi and one for lo.
//
// Packed activation row of length KD (KD % 128 == 0): KD/8 chunks of 32 bytes,
// chunk = [8 fp16 hi | 8 fp16 lo] of columns 8c..8c+7 in the order
// 0,4,1,5,2,6,3,7 (odd columns divided by 16), chunks ordered (step s = c/16,
// word wi = c%4, quarter t = (c/4)%4) so that the four lanes of one row read 64
// contiguous bytes.
#include "sw_common.cuh"
#include <cuda_fp16.h>
#include <stdlib.h>

__device__ __forceinline__ uint4 sw_ldg_stream(const uint4 *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ void sw_mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8 nibbles -> 4 half2 operands: [0]=(n0,n4)*2^-24 [1]=(n1,n5)*2^-20 [2]=(n2,n6)*2^-24 [3]=(n3,n7)*2^-20
__device__ __forceinline__ void sw_dq4(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t w2 = w >> 8;
    h[0] = w & 0x000F000Fu; h[1] = w & 0x00F000F0u;
    h[2] = w2 & 0x000F000Fu; h[3] = w2 & 0x00F000F0u;
}
#define SW_ACC_SCALE 16777216.f      /* 2^24 */

__device__ __forceinline__ uint32_t sw_word(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// position (in halves) of column `col` inside a packed row: chunk*16 + slot
__device__ __forceinline__ size_t sw_packed_pos(int col) {
    const int c8 = col >> 3, s = c8 >> 4, tt = (c8 >> 2) & 3, wi = c8 & 3, j = col & 7;
    return (size_t)(((s * 4 + wi) * 4 + tt) * 16 + ((j & 3) * 2 + (j >> 2)));
}

// f32 -> fp16 hi/lo pair (saturating at the fp16 range); returns the value the pair represents
__device__ __forceinline__ float sw_split_f16(float v, __half &hi, __half &lo) {
    v = fminf(fmaxf(v, -65504.f), 65504.f);
    hi = __float2half_rn(v);
    const float h = __half2float(hi);
    lo = __float2half_rn(v - h);
    return h + __half2float(lo);
}

// ---------------------------------------------------------------------------
// x[rows, KD] f32 -> packed rows + row sums of the represented values.
// One CTA per row; the sum is reduced in double in a fixed order.
// With `rexp` the row is first divided by a power of two 2^e chosen so that its
// largest magnitude lands in [1, 2), and rexp[row] = 2^e: the fp16 pairs then
// carry every row at the same relative precision whatever the caller's scale,
// the gate/up epilogue multiplies the gate back, and SiLU(gate)*up is stored
// divided by 2^2e (the down product multiplies it back), so that no value of
// the pipeline depends on the input's magnitude for its range.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_pack_act(const float *__restrict__ x, uint4 *__restrict__ xp, float *__restrict__ rowsum, int rows, int KD,
           float *__restrict__ rexp, int *__restrict__ status) {
    __shared__ double s_part[8];
    __shared__ float s_max[8];
    bool clamped = false;
    const int cpr = KD >> 3;                                  // chunks per row
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        float inv = 1.f;
        if (rexp) {
            float m = 0.f;
            for (int c8 = threadIdx.x; c8 < cpr; c8 += 256) {
                const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)r * KD + c8 * 8);
                const float4 a = src[0], b = src[1];
                m = fmaxf(m, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                                   fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w)))));
            }
#pragma unroll
            for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(SW_FULL_MASK, m, off));
            __syncthreads();                                  // s_max of the previous row has been read
            if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
            __syncthreads();
            m = s_max[0];
#pragma unroll
            for (int i = 1; i < 8; i++) m = fmaxf(m, s_max[i]);
            float rex = 1.f;
            if (m > 0.f && m <= 3.0e38f) {                    // zero rows, infinities and NaNs keep scale one
                int ex;
                frexpf(m, &ex);                               // m = f * 2^ex, f in [0.5, 1)
                ex = max(-120, min(120, ex - 1));
                rex = ldexpf(1.f, ex); inv = ldexpf(1.f, -ex);
            }
            if (threadIdx.x == 0) rexp[r] = rex;
        }
        double sum = 0.0;
        for (int c8 = threadIdx.x; c8 < cpr; c8 += 256) {
            const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)r * KD + c8 * 8);
            float4 a = src[0], b = src[1];
            a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv; b.x *= inv; b.y *= inv; b.z *= inv; b.w *= inv;
            // order 0,4,1,5,2,6,3,7; odd columns carry 1/16
            const float v[8] = {a.x, b.x, a.y * 0.0625f, b.y * 0.0625f, a.z, b.z, a.w * 0.0625f, b.w * 0.0625f};
            __half hi[8], lo[8];
            float even = 0.f, odd = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                clamped |= !(fabsf(v[i]) <= 65504.f);          // also true for NaN
                const float rep = sw_split_f16(v[i], hi[i], lo[i]);
                if ((i >> 1) & 1) odd += rep; else even += rep;
            }
            sum += (double)even + 16.0 * (double)odd;
            const int s = c8 >> 4, tt = (c8 >> 2) & 3, wi = c8 & 3;
            uint4 *dst = xp + ((size_t)r * cpr + ((s * 4 + wi) * 4 + tt)) * 2;
            dst[0] = *reinterpret_cast<uint4 *>(hi);
            dst[1] = *reinterpret_cast<uint4 *>(lo);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(SW_FULL_MASK, sum, off);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
#pragma unroll
            for (int i = 0; i < 8; i++) t += s_part[i];
            rowsum[r] = (float)t;
        }
    }
    if (clamped && status) atomicOr(status, SW_ST_RANGE);
}

int sw_launch_pack_act(const SwLaunchCfg &c, const float *x, void *xp, float *rowsum, int rows, int KD, float *rexp, int *status) {
    if (rows <= 0) return 0;
    if (KD % 128) return -1;
    int grid = rows < c.num_sms * 8 ? rows : c.num_sms * 8;
    k_pack_act<<<grid, 256, 0, c.stream>>>(x, (uint4 *)xp, rowsum, rows, KD, rexp, status);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// Grouped int4 product.  Warp item = (group, block of MT m-tiles).
//   GATEUP: m-tile = gate rows i..i+7 and up rows I+i..I+i+7, output = packed
//           fp16 hi/lo rows of SiLU(gate)*up  [T*K, I] plus, per packed row and
//           item, the sum of the values it wrote (ypart[row, I/8 slots]), from
//           which the down product rebuilds its row sums in a fixed order
//   else  : m-tile = 16 output rows, output = f32 slots [T*K, D]
// A pass covers 4 token rows (hi|lo side by side) or 8; larger groups loop and
// find the weights of the item in L2.
//
// Weight stream: every thread owns a private ring of P stages in shared memory
// and fills it with 16-byte cp.async copies of the bytes it will itself consume
// (one stage = one 128-column step of its 2*MT rows), so P-1 steps of HBM
// traffic are in flight per thread at no register cost and without any barrier:
// a thread only ever reads back what it copied, after cp.async.wait_group.
//
// Accumulation: the tensor core adds products into its accumulator with
// truncation, which biases a long chain; each 128-column step therefore starts
// from a zero accumulator and is added to the running f32 sum with an ordinary
// round-to-nearest add.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void sw_cp_async16(unsigned smem_addr, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void sw_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void sw_cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// One pass over the contraction for a warp item: streams the 2*MT weight rows
// through the private ring and accumulates MT m-tiles against one n-tile.
// M8: 8 token rows (separate hi and lo MMAs); else 4 rows with hi|lo side by side.
template <int MT, int P, bool M8>
__device__ __forceinline__ void sw_q4_kloop(float (&acc)[MT][4], const uint4 *my, unsigned my_s, const uint4 *wq,
                                            const unsigned (&roff)[2 * MT], const uint4 *xb, int S) {
    constexpr int STAGE = 2 * MT * 128;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt][i] = 0.f;
    // prologue: stages 0..P-2 (one commit per stage keeps the group count uniform)
#pragma unroll
    for (int p = 0; p < P - 1; p++) {
        if (p < S) {
#pragma unroll
            for (int q = 0; q < 2 * MT; q++) sw_cp_async16(my_s + (unsigned)(p * STAGE + q * 128) * 16u, wq + roff[q] + p * 4);
        }
        sw_cp_async_commit();
    }
    int sc = 0, sf = P - 1;                           // ring slot consumed / filled next
    for (int s = 0; s < S; s++) {
        if (s + P - 1 < S) {
#pragma unroll
            for (int q = 0; q < 2 * MT; q++) sw_cp_async16(my_s + (unsigned)(sf * STAGE + q * 128) * 16u, wq + roff[q] + (s + P - 1) * 4);
        }
        sw_cp_async_commit();
        sw_cp_async_wait<P - 1>();                    // stage s has landed
        uint4 wv[2 * MT];
#pragma unroll
        for (int q = 0; q < 2 * MT; q++) wv[q] = my[sc * STAGE + q * 128];
        sc = sc + 1 == P ? 0 : sc + 1;
        sf = sf + 1 == P ? 0 : sf + 1;

        float part[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) part[mt][i] = 0.f;
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            const uint4 *bp = xb + (s * 4 + wi) * 8;
            const uint4 b0 = __ldg(bp);
            uint4 b1;
            if (M8) b1 = __ldg(bp + 1);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                uint32_t ga[4], ua[4];
                sw_dq4(sw_word(wv[2 * mt], wi), ga);
                sw_dq4(sw_word(wv[2 * mt + 1], wi), ua);
                sw_mma_f16(part[mt], ga[0], ua[0], ga[1], ua[1], b0.x, b0.y);
                sw_mma_f16(part[mt], ga[2], ua[2], ga[3], ua[3], b0.z, b0.w);
                if (M8) {
                    sw_mma_f16(part[mt], ga[0], ua[0], ga[1], ua[1], b1.x, b1.y);
                    sw_mma_f16(part[mt], ga[2], ua[2], ga[3], ua[3], b1.z, b1.w);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[mt][i] += part[mt][i];
    }
    sw_cp_async_wait<0>();
}

template <bool GATEUP, int MT, int P>
__global__ void __launch_bounds__(128, (MT == 4 ? 3 : 4))
k_q4_mma(const uint8_t *__restrict__ Wq, const float *__restrict__ Ws,
         const uint4 *__restrict__ XP, const float *__restrict__ xsum, int xsum_parts,
         void *__restrict__ Yout, float *__restrict__ ypart,
         const int *__restrict__ gexp, const int *__restrict__ gbeg, const int *__restrict__ gcnt,
         const int *__restrict__ Gp, const int *__restrict__ grow,
         int KD, int OUT, int expert_lo, int expert_cnt, int *__restrict__ status,
         const float *__restrict__ rex_in, float *__restrict__ srex_out) {
    extern __shared__ uint4 sw_ring[];                        // [P][2*MT][128]
    bool clamped = false;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int warps_total = gridDim.x * 4, wid = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int G = *Gp;
    constexpr int OPI = MT * (GATEUP ? 8 : 16);              // outputs per item
    constexpr int STAGE = 2 * MT * 128;                       // uint4 per ring stage
    const int mb_per_group = (OUT + OPI - 1) / OPI;
    const int items = G * mb_per_group;
    const int S = KD >> 7;                                    // 128-column steps
    const unsigned row_u4 = (unsigned)(KD >> 5);              // uint4 per weight row
    const size_t xrow_u4 = (size_t)(KD >> 2);                 // uint4 per packed activation row
    const int nrows_w = GATEUP ? 2 * OUT : OUT;
    const uint4 *my = sw_ring + threadIdx.x;
    const unsigned my_s = (unsigned)__cvta_generic_to_shared(sw_ring + threadIdx.x);

    for (int item = wid; item < items; item += warps_total) {
        const int gi = item / mb_per_group, mb = item - gi * mb_per_group;
        const int e = gexp[gi] - expert_lo;
        if (e < 0 || e >= expert_cnt) continue;
        const int n = gcnt[gi], beg = gbeg[gi];
        const uint4 *wq = reinterpret_cast<const uint4 *>(Wq) + (size_t)e * nrows_w * row_u4 + t;
        const float *ws = Ws + (size_t)e * nrows_w;

        unsigned roff[2 * MT];                                // [2*mt] = row of role g, [2*mt+1] = row of role g+8
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            int ra, rb;
            if (GATEUP) { int o = min(mb * OPI + mt * 8 + g, OUT - 1); ra = o; rb = OUT + o; }
            else        { int o = mb * OPI + mt * 16 + g; ra = min(o, OUT - 1); rb = min(o + 8, OUT - 1); }
            roff[2 * mt] = (unsigned)ra * row_u4;
            roff[2 * mt + 1] = (unsigned)rb * row_u4;
        }

        for (int c0 = 0; c0 < n;) {
            const bool m8 = n - c0 > 4;                       // warp-uniform: 8 rows (hi, lo apart) or 4 rows (hi|lo)
            const int ntok = m8 ? min(8, n - c0) : n - c0;
            // B column g of this thread: which packed row, and which half of the chunk
            const int bt = m8 ? g : (g & 3);
            const int r = c0 + min(bt, ntok - 1);
            const int rowid = GATEUP ? grow[beg + r] : beg + r;
            const uint4 *xb = XP + (size_t)rowid * xrow_u4 + (size_t)t * 2 + ((!m8 && g >= 4) ? 1 : 0);

            float acc[MT][4];
            if (m8) sw_q4_kloop<MT, P, true>(acc, my, my_s, wq, roff, xb, S);
            else    sw_q4_kloop<MT, P, false>(acc, my, my_s, wq, roff, xb, S);

            // In 4-row mode columns j and j+4 hold the hi and lo parts of one token: fold them.
            if (!m8) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[mt][i] += __shfl_down_sync(SW_FULL_MASK, acc[mt][i], 2);
            }
            // token rows of this thread's two columns, and the "-8 * sum x" correction
            const bool own = m8 || t < 2;
            float corr[2], rex[2]; int tok[2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                tok[j] = c0 + 2 * t + j;
                const bool ok = own && tok[j] < c0 + ntok;
                // row sum of the token's activations: the 8 lanes that share t split the partial
                // sums between them (k = g, g+8, ...) and add up in a fixed tree
                float sx = 0.f;
                rex[j] = 1.f;
                if (ok) {
                    const int rid = GATEUP ? grow[beg + tok[j]] : beg + tok[j];
                    const float *ps = xsum + (size_t)rid * xsum_parts;
                    for (int k = g; k < xsum_parts; k += 8) sx += ps[k];
                    // the power of two the row was divided by (gate/up: the token's; down: the packed row's)
                    if (rex_in) rex[j] = rex_in[rid];
                    if (GATEUP && srex_out && mb == 0 && g == 0) srex_out[beg + tok[j]] = rex[j];
                }
                sx += __shfl_xor_sync(SW_FULL_MASK, sx, 4);
                sx += __shfl_xor_sync(SW_FULL_MASK, sx, 8);
                sx += __shfl_xor_sync(SW_FULL_MASK, sx, 16);
                corr[j] = 8.f * sx;
                if (!ok) tok[j] = -1;
            }

            // epilogue: c[0],c[1] = (row g, tokens 2t,2t+1), c[2],c[3] = (row g+8, same tokens)
            if (GATEUP) {
                float ysum[2] = {0.f, 0.f};
                __half *Y = reinterpret_cast<__half *>(Yout);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const int o = mb * OPI + mt * 8 + g;
                    const bool ov = o < OUT;
                    const float sg = ov ? ws[o] : 0.f, su = ov ? ws[OUT + o] : 0.f;
                    const size_t pos = sw_packed_pos(ov ? o : 0);
                    const float pre = (o & 1) ? 0.0625f : 1.f;
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        if (tok[j] < 0 || !ov) continue;
                        // gate at its true size; the up value stays divided by 2^e and the product is divided once more
                        const float gv = (acc[mt][j] * SW_ACC_SCALE - corr[j]) * sg * rex[j];
                        const float uv = (acc[mt][2 + j] * SW_ACC_SCALE - corr[j]) * su;
                        const float y = ((gv / (1.f + expf(-gv))) * __frcp_rn(rex[j])) * uv;
                        __half hi, lo;
                        clamped |= fabsf(y * pre) > 65504.f;
                        const float rep = sw_split_f16(y * pre, hi, lo);
                        ysum[j] += (o & 1) ? rep * 16.f : rep;
                        __half *row = Y + (size_t)(beg + tok[j]) * (2 * (size_t)OUT);
                        row[pos] = hi; row[pos + 8] = lo;
                    }
                }
                // sum over the item's outputs (the 8 row groups g) in a fixed order
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    float v = ysum[j];
                    v += __shfl_xor_sync(SW_FULL_MASK, v, 4);
                    v += __shfl_xor_sync(SW_FULL_MASK, v, 8);
                    v += __shfl_xor_sync(SW_FULL_MASK, v, 16);
                    if (g == 0 && tok[j] >= 0) ypart[(size_t)(beg + tok[j]) * mb_per_group + mb] = v;
                }
            } else {
                float *Y = reinterpret_cast<float *>(Yout);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const int oa = mb * OPI + mt * 16 + g, ob = oa + 8;
                    const float sa = oa < OUT ? ws[oa] : 0.f, sb = ob < OUT ? ws[ob] : 0.f;
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        if (tok[j] < 0) continue;
                        float *row = Y + (size_t)(beg + tok[j]) * OUT;
                        const float back = rex[j] * rex[j];             // SiLU(gate)*up came in divided by 2^2e
                        if (oa < OUT) row[oa] = (acc[mt][j] * SW_ACC_SCALE - corr[j]) * sa * back;
                        if (ob < OUT) row[ob] = (acc[mt][2 + j] * SW_ACC_SCALE - corr[j]) * sb * back;
                    }
                }
            }
            c0 += ntok;
        }
    }
    if (GATEUP && clamped && status) atomicOr(status, SW_ST_RANGE);
}

template <bool GATEUP, int MT, int P>
static int sw_launch_q4_mma_t(const SwLaunchCfg &c, const SwQ4Args &a, const SwMmaIO &io) {
    static SwPerDevice per_dev;                       // resident CTAs per SM of this instantiation, per device
    constexpr int SMEM = P * 2 * MT * 128 * 16;
    auto kern = k_q4_mma<GATEUP, MT, P>;
    const int ctas_per_sm = per_dev.get(c.dev, [&] {
        int n = 0;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 128, SMEM) != cudaSuccess || n < 1) { cudaGetLastError(); n = 1; }
        return n; });
    if (ctas_per_sm <= 0) return -1;
    long long grid = (long long)c.num_sms * ctas_per_sm;
    constexpr int OPI = MT * (GATEUP ? 8 : 16);
    long long items = (long long)a.max_groups * ((a.OUT + OPI - 1) / OPI);
    long long need = (items + 3) / 4;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, 128, SMEM, c.stream>>>(a.q, a.s, (const uint4 *)io.XP, io.xsum, io.xsum_parts, io.Y, io.ypart,
                                                  a.gexp, a.gbeg, a.gcnt, a.G, a.grow, a.KD, a.OUT, a.expert_lo, a.expert_cnt, io.status, io.rex, io.srex_out);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// m-tiles per warp item for a launch: few groups (single-row decode) want small
// items so that every SM gets work; SW_MMA_MT=1|2|4 overrides the choice (tuning knob).
int sw_q4_mma_mt(const SwLaunchCfg &c, const SwQ4Args &a, bool gateup) {
    const int mt_env = sw_tuning().mma_mt;
    if (mt_env == 1 || mt_env == 2 || mt_env == 4) return mt_env;
    const int opi4 = gateup ? 32 : 64;
    const long long items4 = (long long)a.max_groups * ((a.OUT + opi4 - 1) / opi4);
    return items4 >= (long long)c.num_sms * 32 ? 4 : items4 >= (long long)c.num_sms * 8 ? 2 : 1;
}

// io.XP: packed activation rows (gate/up: the token rows, indexed through grow;
// down: the packed SiLU*up rows) with io.xsum[row, xsum_parts] partial row sums.
// io.Y: gate/up -> packed rows [max_rows, OUT] and io.ypart[max_rows, OUT/(8*mt)]; down -> f32.
int sw_launch_q4_mma(const SwLaunchCfg &c, const SwQ4Args &a, const SwMmaIO &io, bool gateup, int mt) {
    if (a.max_groups <= 0 || a.max_rows <= 0) return 0;
    if (a.KD % 128 || a.OUT <= 0) return -1;
    if (gateup) return mt == 4 ? sw_launch_q4_mma_t<true, 4, 4>(c, a, io) : mt == 2 ? sw_launch_q4_mma_t<true, 2, 6>(c, a, io) : sw_launch_q4_mma_t<true, 1, 12>(c, a, io);
    return mt == 4 ? sw_launch_q4_mma_t<false, 4, 4>(c, a, io) : mt == 2 ? sw_launch_q4_mma_t<false, 2, 6>(c, a, io) : sw_launch_q4_mma_t<false, 1, 12>(c, a, io);
}

// ===========================================================================
// bf16 shared expert on the tensor cores.
//
// Weights are bf16 and go into the A fragments as they are (a thread's 16
// bytes of a row are 8 consecutive columns = the k-slots of two MMAs), the
// activations are split into two bf16 terms (x = hi + lo to 16 bits) stored
// row-major as 32-byte chunks [8 hi | 8 lo] per 8 columns.  Rows g / g+8 of an
// m-tile are gate row i and up row i (SiLU(gate)*up is thread-local) or two
// output rows of the down projection.  Up to 32 token rows per pass.
// Reference contract: matmul_bf16_k round_x=0 (c/moe_matmul.h:92-111) and
// lag_shared (c/laguna.c:596-602).
// ===========================================================================
__device__ __forceinline__ void sw_mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void sw_split_bf16(float v, __nv_bfloat16 &hi, __nv_bfloat16 &lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// x[rows, KD] f32 -> rows of KD/8 chunks [8 bf16 hi | 8 bf16 lo]
__global__ void __launch_bounds__(256)
k_pack_bf16(const float *__restrict__ x, uint4 *__restrict__ xp, int rows, int KD) {
    const int cpr = KD >> 3;
    const size_t n = (size_t)rows * cpr;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const float4 *src = reinterpret_cast<const float4 *>(x) + idx * 2;
        const float4 a = src[0], b = src[1];
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        __nv_bfloat16 hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) sw_split_bf16(v[i], hi[i], lo[i]);
        xp[idx * 2] = *reinterpret_cast<uint4 *>(hi);
        xp[idx * 2 + 1] = *reinterpret_cast<uint4 *>(lo);
    }
}

int sw_launch_pack_bf16(const SwLaunchCfg &c, const float *x, void *xp, int rows, int KD) {
    if (rows <= 0) return 0;
    if (KD % 8) return -1;
    size_t n = (size_t)rows * (KD / 8);
    long long grid = (long long)((n + 255) / 256);
    if (grid > (long long)c.num_sms * 8) grid = (long long)c.num_sms * 8;
    k_pack_bf16<<<(unsigned)grid, 256, 0, c.stream>>>(x, (uint4 *)xp, rows, KD);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// KD % 32 == 0.  Warp item = (block of 16 weight rows, slice of the contraction);
// the f32 partial sums of a slice go to Ypart[slice][token][OW] (OW = 2*O for
// gate/up: gate at o, up at O+o; OW = O for down) and are added in slice order by
// the consumer (k_shared_glu / the combine), which keeps every tensor-core
// accumulation chain short and the result independent of scheduling.  The weight
// rows stream through a per-thread cp.async ring like the int4 kernel.
template <bool GATEUP, int P>
__global__ void __launch_bounds__(128)
k_bf16_mma(const __nv_bfloat16 *__restrict__ W0, const __nv_bfloat16 *__restrict__ W1,
           const uint4 *__restrict__ XP, float *__restrict__ Ypart, int T, int KD, int O, int KS, int slice) {
    extern __shared__ uint4 sw_ring[];                        // [P][2][128]
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int warps_total = gridDim.x * 4, wid = blockIdx.x * 4 + (threadIdx.x >> 5);
    constexpr int OPI = GATEUP ? 8 : 16;
    const int mblocks = (O + OPI - 1) / OPI;
    const int items = mblocks * KS;
    const size_t row_u4 = (size_t)(KD >> 3);                  // uint4 per weight row
    const size_t xrow_u4 = (size_t)(KD >> 2);                 // uint4 per packed activation row
    const int OW = GATEUP ? 2 * O : O;
    constexpr int NTM = 4;                                    // n-tiles per pass
    const uint4 *my = sw_ring + threadIdx.x;
    const unsigned my_s = (unsigned)__cvta_generic_to_shared(sw_ring + threadIdx.x);

    for (int item = wid; item < items; item += warps_total) {
        const int ks = item % KS, mb = item / KS;
        const int s0 = (ks * slice) >> 5, s1 = min(KD, (ks + 1) * slice) >> 5;   // 32-column steps [s0, s1)
        const int S = s1 - s0;
        const uint4 *pa, *pb;
        if (GATEUP) {
            const int o = min(mb * 8 + g, O - 1);
            pa = reinterpret_cast<const uint4 *>(W0) + (size_t)o * row_u4 + t + (size_t)s0 * 4;
            pb = reinterpret_cast<const uint4 *>(W1) + (size_t)o * row_u4 + t + (size_t)s0 * 4;
        } else {
            const int o = mb * 16 + g;
            pa = reinterpret_cast<const uint4 *>(W0) + (size_t)min(o, O - 1) * row_u4 + t + (size_t)s0 * 4;
            pb = reinterpret_cast<const uint4 *>(W0) + (size_t)min(o + 8, O - 1) * row_u4 + t + (size_t)s0 * 4;
        }
        for (int c0 = 0; c0 < T; c0 += 8 * NTM) {
            const int nt_used = min(NTM, (T - c0 + 7) >> 3);  // warp-uniform
            const uint4 *xb[NTM];
#pragma unroll
            for (int nt = 0; nt < NTM; nt++) xb[nt] = XP + (size_t)min(c0 + nt * 8 + g, T - 1) * xrow_u4 + (size_t)t * 2 + (size_t)s0 * 8;
            float acc[NTM][4];
#pragma unroll
            for (int nt = 0; nt < NTM; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[nt][i] = 0.f;

#pragma unroll
            for (int p = 0; p < P - 1; p++) {
                if (p < S) { sw_cp_async16(my_s + (unsigned)(p * 256) * 16u, pa + p * 4); sw_cp_async16(my_s + (unsigned)(p * 256 + 128) * 16u, pb + p * 4); }
                sw_cp_async_commit();
            }
            int sc = 0, sf = P - 1;
            for (int s = 0; s < S; s++) {
                if (s + P - 1 < S) {
                    sw_cp_async16(my_s + (unsigned)(sf * 256) * 16u, pa + (s + P - 1) * 4);
                    sw_cp_async16(my_s + (unsigned)(sf * 256 + 128) * 16u, pb + (s + P - 1) * 4);
                }
                sw_cp_async_commit();
                sw_cp_async_wait<P - 1>();
                const uint4 wa = my[sc * 256], wb = my[sc * 256 + 128];
                sc = sc + 1 == P ? 0 : sc + 1;
                sf = sf + 1 == P ? 0 : sf + 1;
#pragma unroll
                for (int nt = 0; nt < NTM; nt++) {
                    if (nt < nt_used) {
                        const uint4 bh = __ldg(xb[nt] + (size_t)s * 8), bl = __ldg(xb[nt] + (size_t)s * 8 + 1);
                        sw_mma_bf16(acc[nt], wa.x, wb.x, wa.y, wb.y, bh.x, bh.y);
                        sw_mma_bf16(acc[nt], wa.z, wb.z, wa.w, wb.w, bh.z, bh.w);
                        sw_mma_bf16(acc[nt], wa.x, wb.x, wa.y, wb.y, bl.x, bl.y);
                        sw_mma_bf16(acc[nt], wa.z, wb.z, wa.w, wb.w, bl.z, bl.w);
                    }
                }
            }
            sw_cp_async_wait<0>();
            // c[0],c[1] = (row g, tokens 2t,2t+1); c[2],c[3] = (row g+8, same tokens)
            const int oa = GATEUP ? mb * 8 + g : mb * 16 + g;
            const int ob = GATEUP ? O + oa : oa + 8;
            const bool va = oa < O, vb = GATEUP ? va : ob < O;
#pragma unroll
            for (int nt = 0; nt < NTM; nt++) {
                if (nt >= nt_used) continue;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int tok = c0 + nt * 8 + 2 * t + j;
                    if (tok >= T) continue;
                    float *row = Ypart + ((size_t)ks * T + tok) * OW;
                    if (va) row[oa] = acc[nt][j];
                    if (vb) row[ob] = acc[nt][2 + j];
                }
            }
        }
    }
}

// sglu packed rows [T, SI] (bf16 hi|lo chunks) = SiLU(sum_ks gate) * (sum_ks up)
__global__ void __launch_bounds__(256)
k_shared_glu(const float *__restrict__ part, int KS, int T, int SI, uint4 *__restrict__ out) {
    const int cpr = SI >> 3;
    const size_t n = (size_t)T * cpr;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int tok = (int)(idx / cpr), c8 = (int)(idx - (size_t)tok * cpr);
        float gv[8], uv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { gv[i] = 0.f; uv[i] = 0.f; }
        for (int ks = 0; ks < KS; ks++) {
            const float4 *pg = reinterpret_cast<const float4 *>(part + ((size_t)ks * T + tok) * (2 * (size_t)SI) + c8 * 8);
            const float4 *pu = reinterpret_cast<const float4 *>(part + ((size_t)ks * T + tok) * (2 * (size_t)SI) + SI + c8 * 8);
            const float4 a = pg[0], b = pg[1], c = pu[0], d = pu[1];
            gv[0] += a.x; gv[1] += a.y; gv[2] += a.z; gv[3] += a.w; gv[4] += b.x; gv[5] += b.y; gv[6] += b.z; gv[7] += b.w;
            uv[0] += c.x; uv[1] += c.y; uv[2] += c.z; uv[3] += c.w; uv[4] += d.x; uv[5] += d.y; uv[6] += d.z; uv[7] += d.w;
        }
        __nv_bfloat16 hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) sw_split_bf16((gv[i] / (1.f + expf(-gv[i]))) * uv[i], hi[i], lo[i]);
        out[idx * 2] = *reinterpret_cast<uint4 *>(hi);
        out[idx * 2 + 1] = *reinterpret_cast<uint4 *>(lo);
    }
}

// Slices of the contraction for a shared-expert product with `mblocks` row blocks.
int sw_shared_slices(int num_sms, int mblocks, int KD) {
    int want = (num_sms * 12 + mblocks - 1) / mblocks;
    int maxs = KD / 256 > 0 ? KD / 256 : 1;
    return want < 1 ? 1 : want > maxs ? maxs : want;
}

// Shared expert product: XP = packed rows (k_pack_bf16 / k_shared_glu); part = f32 [KS][T][OW].
int sw_launch_bf16_mma(const SwLaunchCfg &c, const void *W0, const void *W1, const void *XP, float *part,
                       int T, int KD, int O, int KS, bool gateup) {
    if (T <= 0 || O <= 0) return 0;
    if (KD % 32 || KS < 1) return -1;
    constexpr int P = 8;
    constexpr int SMEM = P * 2 * 128 * 16;
    static SwPerDevice attr;
    if (attr.get(c.dev, [] {
            if (cudaFuncSetAttribute(k_bf16_mma<true, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
                cudaFuncSetAttribute(k_bf16_mma<false, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    const int mblocks = (O + (gateup ? 8 : 16) - 1) / (gateup ? 8 : 16);
    const int slice = ((KD + KS - 1) / KS + 31) & ~31;
    long long items = (long long)mblocks * KS, need = (items + 3) / 4;
    long long grid = (long long)c.num_sms * 4;
    if (grid > need) grid = need;
    if (gateup) k_bf16_mma<true, P><<<(unsigned)grid, 128, SMEM, c.stream>>>((const __nv_bfloat16 *)W0, (const __nv_bfloat16 *)W1, (const uint4 *)XP, part, T, KD, O, KS, slice);
    else k_bf16_mma<false, P><<<(unsigned)grid, 128, SMEM, c.stream>>>((const __nv_bfloat16 *)W0, nullptr, (const uint4 *)XP, part, T, KD, O, KS, slice);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int sw_launch_shared_glu(const SwLaunchCfg &c, const float *part, int KS, int T, int SI, void *out) {
    if (T <= 0) return 0;
    if (SI % 8) return -1;
    size_t n = (size_t)T * (SI / 8);
    long long grid = (long long)((n + 255) / 256);
    if (grid > (long long)c.num_sms * 8) grid = (long long)c.num_sms * 8;
    k_shared_glu<<<(unsigned)grid, 256, 0, c.stream>>>(part, KS, T, SI, (uint4 *)out);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
