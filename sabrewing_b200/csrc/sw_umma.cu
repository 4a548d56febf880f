// Grouped int4 expert GEMM on the 5th-generation tensor cores (tcgen05 + TMEM)
// for groups with many token rows (prefill, large decode batches).
//
// D[weight rows, token rows] = W . X^T: 128 dequantised weight rows are the A operand
// (M = 128), a chunk of <= 128 token rows of one expert group (padded to 16/32/64/128)
// the B operand, f32 accumulators in tensor memory.  A CTA work item is a chunk times
// a PAIR of weight tiles that share the chunk's activation tiles (gate/up: the gate
// rows of 128 outputs and their up rows, so SiLU(gate)*up is lane-local in the
// epilogue; down: two neighbouring tiles).  K runs in steps of 128 columns.  Fifteen
// warps, four roles:
//   warp 12      TMA producer: per step the raw int4 rows of both tiles (2 x 128 rows x
//                64 B, 64-byte swizzle) and the fp16 activation tiles (two 64-column
//                sub-tiles of R rows x 128 B per term, 128B swizzle = the K-major
//                canonical layout the tensor core reads) into a ring of four 48-KB slots
//                (two 80-KB slots with two terms)
//   warps 0-7    dequantise, two groups of four: a thread owns one row of tile t, reads
//                its 64 raw bytes of the step from the slot, expands them to 128 exact
//                fp16 integers (nibble - 8) in registers and stores them with tcgen05.st
//                into one of four A tiles in TENSOR MEMORY (64 columns each)
//   warps 13,14  MMA issuers, one per tile of the pair: eight tcgen05.mma kind::f16 per
//                step with the A operand in tensor memory and B through its
//                shared-memory descriptor (with two terms a second MMA against the lo
//                tile into the same accumulator columns); two tcgen05.commit per step:
//                one returns the A tile to its tile's dequantising warps, one (counted
//                from both issuers) the slot to the TMA warp.  The WHOLE warp runs the loop
//                with warp-uniform values and an elected lane issues (elect.sync), so
//                that the descriptors are computed in uniform registers
//   warps 8-11   epilogue: tcgen05.ld the two accumulators of the item, apply the per-row
//                scales and SiLU(gate)*up, or store the f32 slot rows.  The accumulators
//                have ONE buffer (tensor memory: 256 columns of accumulators + 256 of A
//                tiles), so the dequantising warps, idle at that point, take two thirds
//                of every item's epilogue.
// Why the A operand sits in tensor memory: with both operands in shared memory an
// M = 128, N = 128, K = 16 MMA reads 8 KB in its 64 cycles, all the shared-memory
// bandwidth of an SM, and the dequantised tiles crossed it once more on their way in.
//
// Activations are fp16 arrays [rows, K] whose columns are permuted inside every group
// of eight to 0,4,1,5,2,6,3,7 -- the order in which the nibble masks deliver a weight
// word -- so the K order of a dequantised row matches.  `terms` = 1 feeds the tensor
// core fp16(x) alone (relative rounding 2^-12 per element); `terms` = 2 adds the
// residual lo = fp16(x - hi) as a second MMA per step (f32-level accuracy, twice the
// tensor work).  The token rows of gate/up are gathered into packed-slot order by
// k_umma_gather (the reference gathers too, c/laguna.c:742-743).
//
// All mbarrier waits are bounded; on a timeout the CTA raises an abort flag, sets
// SW_ST_TIMEOUT in the status word and still frees its tensor memory.
#include "sw_common.cuh"
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#define UM_RAW_A 8192                    // raw int4 of one weight tile and step: 128 rows x 64 B (128 columns)
#define UM_BT 16384                      // one activation sub-tile: 128 rows x 128 B (64 columns)
#define UM_WAIT_LIMIT (1u << 24)
// K runs in steps of 128 columns.  A ring slot holds, for one step, the raw int4 rows of a pair of weight tiles
// (2 x 8 KB, 64-byte rows under the 64-byte TMA swizzle so that a thread reads its row without bank conflicts) and
// the fp16 activation tiles they share (two 64-column sub-tiles of 16 KB per term): 48 KB with one term (four
// slots), 80 KB with two (two slots).  The dequantised weight tiles do NOT live in shared memory: they go from
// registers into tensor memory (tcgen05.st) and the MMAs take their A operand from there.  With both operands in
// shared memory an M = 128, N = 128, K = 16 MMA reads 8 KB in its 64 cycles, which is all the shared-memory
// bandwidth an SM has (128 B/cycle), and the dequantised tiles crossed it a second time on their way in.
#define UM_STAGE_BYTES(terms) (2 * UM_RAW_A + 2 * (terms) * UM_BT)
#define UM_STAGES_FOR(terms) ((terms) == 1 ? 4 : 2)
#define UM_MAX_STAGES 8
#define UM_RING_BYTES (4 * UM_STAGE_BYTES(1))        // 192 KB: four slots of 48 KB, or two of 80 KB
// Tensor memory (512 columns): the two accumulators of an item in columns [0, 256) (one buffer), and a ring of four
// dequantised A tiles -- two steps of a tile pair, 64 columns each (128 rows x 128 fp16) -- in columns [256, 512).
#define UM_A_SLOTS 2
#define UM_ABUF (2 * UM_A_SLOTS)
#define UM_TMEM_A 256
#define UM_DQ_WARPS 8                              // dequantise (and two thirds of the epilogue): two per tensor-memory lane quarter
#define UM_EPI_WARPS 4                             // epilogue only: one per lane quarter
#define UM_WARP_TMA (UM_DQ_WARPS + UM_EPI_WARPS)
#define UM_WARP_MMA (UM_WARP_TMA + 1)              // and UM_WARP_MMA + 1
#define UM_THREADS ((UM_WARP_MMA + 2) * 32)

__device__ __forceinline__ unsigned um_s32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void um_bar_init(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void um_bar_expect(unsigned bar, unsigned bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void um_bar_arrive(unsigned bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ bool um_bar_wait(unsigned bar, unsigned parity, volatile int *abortp) {
    for (unsigned it = 0; it < UM_WAIT_LIMIT; it++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 255) == 255 && *abortp) return false;
    }
    return false;
}
__device__ __forceinline__ void um_tma_2d(unsigned dst, const CUtensorMap *tm, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar) : "memory");
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t um_desc(unsigned saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);            // start address
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset
    d |= (uint64_t)1 << 46;                             // descriptor version
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}
// tcgen05.mma, executed by a whole warp with warp-uniform operands: one elected lane issues (and the same lane
// issues the commits, which track the operations of the thread that executes them).  Keeping the issuing code
// warp-uniform lets the descriptors live in uniform registers, which is where the instruction takes them from; computed
// per thread (inside an `if (lane == 0)`) every operand of every MMA is first moved across, and the moves, not the tensor
// pipe, set the issue rate (measured: 190 against 64 clocks per M = 128, N = 128, K = 16 MMA).
// A operand in tensor memory (128 lanes x 8 columns of two fp16 each per K = 16), B through its shared-memory descriptor;
// the election is done once by the caller (um_elect): `leader` is 1 in the elected lane, 0 elsewhere
__device__ __forceinline__ unsigned um_elect() {
    unsigned l;
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\tselp.u32 %0, 1, 0, e;\n\t}" : "=r"(l));
    return l;
}
__device__ __forceinline__ void um_mma_ta_lead(unsigned leader, unsigned d_tmem, unsigned a_tmem, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p, e;\n\tsetp.ne.b32 e, %5, 0;\n\tsetp.ne.b32 p, %4, 0;\n\t@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
}
__device__ __forceinline__ void um_commit_lead(unsigned leader, unsigned bar) {
    asm volatile("{\n\t.reg .pred e;\n\tsetp.ne.b32 e, %1, 0;\n\t@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" :: "r"(bar), "r"(leader) : "memory");
}
// both operands through shared-memory descriptors, election per instruction
__device__ __forceinline__ void um_mma_elect(unsigned d_tmem, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p, e;\n\telect.sync _|e, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void um_commit_elect(unsigned bar) {
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" :: "r"(bar) : "memory");
}
// 16 consecutive columns of this thread's lane (the caller waits with tcgen05.wait::st)
__device__ __forceinline__ void um_st16_nowait(unsigned taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                    "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void um_ld32(unsigned taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void um_ld16(unsigned taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
// 8 nibbles -> 8 fp16 (nibble-8) in the order c0,c4,c1,c5,c2,c6,c3,c7
__device__ __forceinline__ uint4 um_dq(uint32_t w) {
    const uint32_t MAGIC = 0x64006400u, C1032 = 0x64086408u, C16TH = 0x2C002C00u, CM72 = 0xD480D480u;
    const uint32_t l0 = (w & 0x000F000Fu) | MAGIC, h0 = (w & 0x00F000F0u) | MAGIC;
    const uint32_t w2 = w >> 8;
    const uint32_t l1 = (w2 & 0x000F000Fu) | MAGIC, h1 = (w2 & 0x00F000F0u) | MAGIC;
    uint4 o;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(o.x) : "r"(l0), "r"(C1032));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(o.y) : "r"(h0), "r"(C16TH), "r"(CM72));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(o.z) : "r"(l1), "r"(C1032));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(o.w) : "r"(h1), "r"(C16TH), "r"(CM72));
    return o;
}
__device__ __forceinline__ int um_perm8(int col) { const int j = col & 7; return (col & ~7) | ((j & 3) * 2 + (j >> 2)); }
__device__ __forceinline__ void um_split(float v, __half &hi, __half &lo) {
    v = fminf(fmaxf(v, -65504.f), 65504.f);
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}

// ---------------------------------------------------------------------------
// xg_hi/xg_lo[slot, :] = fp16 hi/lo of x[grow[slot], :] with the columns of each
// group of eight in the order 0,4,1,5,2,6,3,7
// ---------------------------------------------------------------------------
// rexp[row] = the power of two 2^e with max|x[row, :]| / 2^e in [1, 2) (1 for rows of zeros, infinities, NaNs).
// One warp per row.  The gather divides every token row by it, so that the fp16 planes carry all rows at the same relative
// precision whatever the caller's scale; the epilogues multiply back (see k_pack_act, which does the same for the decode kernels).
__global__ void __launch_bounds__(256)
k_row_exp(const float *__restrict__ x, int rows, int KD, float *__restrict__ rexp) {
    const int lane = threadIdx.x & 31;
    for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += gridDim.x * 8) {
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)r * KD);
        float m = 0.f;
        for (int i = lane; i < (KD >> 2); i += 32) {
            const float4 a = src[i];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float rex = 1.f;
        if (m > 0.f && m <= 3.0e38f) {
            int ex;
            frexpf(m, &ex);
            rex = ldexpf(1.f, max(-120, min(120, ex - 1)));
        }
        if (lane == 0) rexp[r] = rex;
    }
}

__global__ void __launch_bounds__(256)
k_umma_gather(const float *__restrict__ x, const int *__restrict__ grow, const int *__restrict__ npairs, int P, int KD,
              __half *__restrict__ hi, __half *__restrict__ lo, int *__restrict__ status,
              const float *__restrict__ rexp, float *__restrict__ srex) {
    const int cpr = KD >> 3;
    P = min(P, *npairs);                         // packed rows the dispatch filled (pairs that selected no expert leave none)
    bool clamped = false;
    // a warp per packed row: the row's token and power of two are fetched once, then the lanes walk the row's 8-column
    // chunks four at a time (eight independent 16-byte loads in flight per lane)
    const int lane = threadIdx.x & 31;
    for (int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); slot < P; slot += gridDim.x * (blockDim.x >> 5)) {
        const int tokrow = grow[slot];
        float inv = 1.f;
        if (rexp) {
            const float rex = rexp[tokrow];
            inv = __frcp_rn(rex);                                  // a power of two: exact
            if (lane == 0) srex[slot] = rex;                       // the packed row's copy, for the epilogues
        }
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)tokrow * KD);
        uint4 *dh = reinterpret_cast<uint4 *>(hi) + (size_t)slot * cpr;
        uint4 *dl = lo ? reinterpret_cast<uint4 *>(lo) + (size_t)slot * cpr : nullptr;
        for (int c0 = lane; c0 < cpr; c0 += 128) {
            float4 a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c8 = c0 + 32 * u;
                if (c8 < cpr) { a[u] = src[2 * c8]; b[u] = src[2 * c8 + 1]; }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c8 = c0 + 32 * u;
                if (c8 >= cpr) continue;
                const float v[8] = {a[u].x * inv, b[u].x * inv, a[u].y * inv, b[u].y * inv, a[u].z * inv, b[u].z * inv, a[u].w * inv, b[u].w * inv};
                __half h[8], l[8];
#pragma unroll
                for (int i = 0; i < 8; i++) { clamped |= !(fabsf(v[i]) <= 65504.f); um_split(v[i], h[i], l[i]); }
                dh[c8] = *reinterpret_cast<uint4 *>(h);
                if (dl) dl[c8] = *reinterpret_cast<uint4 *>(l);
            }
        }
    }
    if (clamped && status) atomicOr(status, SW_ST_RANGE);
}

// work list: one entry per (group, chunk of <= cap rows): {group index, first row of the chunk inside the group}
__global__ void __launch_bounds__(1024)
k_umma_chunks(const int *__restrict__ Gp, const int *__restrict__ gexp, const int *__restrict__ gcnt,
              int expert_lo, int expert_cnt, int *__restrict__ nchunks, int2 *__restrict__ chunks, int cap) {
    __shared__ int s_scan[1024];
    const int G = *Gp, tid = threadIdx.x;
    int c = 0;
    if (tid < G) { const int e = gexp[tid] - expert_lo; if (e >= 0 && e < expert_cnt) c = (gcnt[tid] + cap - 1) / cap; }
    s_scan[tid] = c;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
        int v = tid >= off ? s_scan[tid - off] : 0;
        __syncthreads();
        s_scan[tid] += v;
        __syncthreads();
    }
    const int base = s_scan[tid] - c;
    for (int i = 0; i < c; i++) chunks[base + i] = make_int2(tid, i * cap);
    if (tid == 1023) *nchunks = s_scan[1023];
}

struct UmArgs {
    const float *Ws;
    void *Y0, *Y1;                 // gate/up: fp16 hi, lo [rows, OUT] (permuted columns); down: f32 slots [rows, OUT], unused
    const int *gexp, *gbeg, *gcnt, *nchunks;
    const int2 *chunks;
    int *status;
    int KD, OUT, expert_lo;
    int terms;                     // fp16 terms per activation: 1 = hi only, 2 = hi + lo
    const float *srex;             // per packed row: the power of two its token row was divided by (null = 1)
    // Ring geometry.  Large groups: chunks of up to 128 rows, 4 slots of 48 KB (2 of 80 KB with two terms).  Small groups
    // (a launch whose groups average at most 32 rows): chunks of up to 32 rows, so that the activation tiles are 8 KB and
    // the ring has 8 slots of 24 KB (6 of 32 KB) -- the weights of such a launch come cold from HBM, and the bytes in
    // flight per SM, not the arithmetic, set its speed.
    int chunk_rows, stages, stage_bytes;
};

template <bool GATEUP>
__global__ void __launch_bounds__(UM_THREADS, 1)
k_q4_umma(const __grid_constant__ CUtensorMap tmW,
          const __grid_constant__ CUtensorMap tmH16, const __grid_constant__ CUtensorMap tmH32,
          const __grid_constant__ CUtensorMap tmH64, const __grid_constant__ CUtensorMap tmH128,
          const __grid_constant__ CUtensorMap tmL16, const __grid_constant__ CUtensorMap tmL32,
          const __grid_constant__ CUtensorMap tmL64, const __grid_constant__ CUtensorMap tmL128,
          const UmArgs a) {
    extern __shared__ unsigned char um_dyn[];
    __shared__ unsigned long long b_raw_full[UM_MAX_STAGES], b_raw_free[UM_MAX_STAGES], b_a_full[UM_ABUF], b_a_free[UM_ABUF], b_acc_full[2], b_acc_free;
    __shared__ unsigned s_tmem;
    __shared__ int s_abort;
    // the powers of two of the item's (<= 128) packed rows, left here by the epilogue warps while the item's MMAs run
    // (two buffers: the dequantising warps may still be reading one item's when the next item's are fetched)
    // [0]: 2^e of each row; [1]: 2^-e (gate/up only: the down product leaves its rows divided by 2^2e for the combine step)
    __shared__ __align__(16) float s_srex[2][2][128];
    __shared__ unsigned long long b_srex[2];
    unsigned char *smem = (unsigned char *)(((uintptr_t)um_dyn + 1023) & ~(uintptr_t)1023);
    const unsigned STG = a.stages, SBYTES = a.stage_bytes;               // ring depth and slot size
    const int CR = a.chunk_rows;                                         // rows per chunk at most
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KD = a.KD, OUT = a.OUT;
    const int nrows_w = GATEUP ? 2 * OUT : OUT;
    // A CTA item is a chunk of token rows times a PAIR of 128-row weight tiles that share the chunk's activation tiles:
    // gate/up: the gate rows of 128 outputs and their up rows; down: two neighbouring tiles (256 outputs).
    constexpr int OPP = GATEUP ? 128 : 256;                             // outputs per pair
    const int pairs = OUT / OPP;
    const int NST = KD >> 7;                                            // 128-column steps per tile
    const int items = *a.nchunks * pairs;
    volatile int *abortp = &s_abort;

    if (threadIdx.x == 0) {
        for (int i = 0; i < UM_MAX_STAGES; i++) { um_bar_init(um_s32(&b_raw_full[i]), 1); um_bar_init(um_s32(&b_raw_free[i]), 2); }
        for (int i = 0; i < UM_ABUF; i++) { um_bar_init(um_s32(&b_a_full[i]), UM_DQ_WARPS / 2); um_bar_init(um_s32(&b_a_free[i]), 1); }
        for (int i = 0; i < 2; i++) um_bar_init(um_s32(&b_acc_full[i]), 1);
        for (int i = 0; i < 2; i++) um_bar_init(um_s32(&b_srex[i]), UM_EPI_WARPS);
        um_bar_init(um_s32(&b_acc_free), UM_DQ_WARPS + UM_EPI_WARPS);   // the epilogue warps and the dequantising warps, which take shares of it
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == UM_WARP_MMA) {                                          // all 512 columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(um_s32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = s_tmem;

    // item -> (chunk, tile pair): the pairs of one chunk are neighbours, so its activation rows stay in L2
    auto decode = [&](int item, int &gi, int &c0, int &pr) {
        const int ch = item / pairs; pr = item - ch * pairs;
        const int2 c = a.chunks[ch]; gi = c.x; c0 = c.y;
    };

    // Slot layout: [raw int4 of the tile pair: 256 rows x 32 B][hi tile: R x 128 B][lo tile: R x 128 B].
    // Raw rows: the 128 rows of tile 0 (gate rows), then the 128 rows of tile 1 (up rows).
    auto tile_rows = [](int n) { return n <= 16 ? 16 : n <= 32 ? 32 : n <= 64 ? 64 : 128; };
    const bool two_terms = a.terms == 2;

    // The epilogue of an item, shared by three warps per tensor-memory lane quarter (the quarter's epilogue warp and its
    // two dequantising warps, which have nothing to dequantise until the accumulators are free again): blocks of 16
    // token columns are dealt round robin, share `part` of 3.  There is one accumulator buffer, so this time is not
    // hidden under MMAs: it has to be short.
    auto epilogue_share = [&](int item, unsigned nitem, int part, bool &clamped) -> bool {
        const int q = warp & 3, trow = q * 32 + lane;                   // lane quarter of this warp, tile row of this thread
        int gi, c0, pr; decode(item, gi, c0, pr);
        const int e = a.gexp[gi] - a.expert_lo, n = min(CR, a.gcnt[gi] - c0), row0 = a.gbeg[gi] + c0;
        const float *ws = a.Ws + (size_t)e * nrows_w;
        if (!um_bar_wait(um_s32(&b_acc_full[0]), nitem & 1, abortp) ||
            !um_bar_wait(um_s32(&b_acc_full[1]), nitem & 1, abortp)) {
            if (lane == 0) { atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; }
            return false;
        }
        if (GATEUP && !um_bar_wait(um_s32(&b_srex[nitem & 1]), (nitem >> 1) & 1, abortp)) {
            if (lane == 0) { atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; }
            return false;
        }
        const float4 *srex4 = reinterpret_cast<const float4 *>(s_srex[nitem & 1][0]);
        const float4 *saux4 = reinterpret_cast<const float4 *>(s_srex[nitem & 1][1]);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned t0 = tmem + ((unsigned)(q * 32) << 16), t1 = t0 + 128;   // tile 0 / tile 1 of this lane
        if (GATEUP) {
            // lane r holds gate row r in tile 0 and up row r in tile 1: output o = pair*128 + r
            const int o = pr * 128 + trow;
            const float sg = o < OUT ? ws[o] : 0.f, su = o < OUT ? ws[OUT + o] : 0.f;
            __half *Yh = reinterpret_cast<__half *>(a.Y0), *Yl = reinterpret_cast<__half *>(a.Y1);
            const int pcol = um_perm8(o);
            // This loop is not hidden under MMAs (one accumulator buffer) and it is instruction-bound, so it is kept short:
            // fast exp and reciprocal (SiLU to ~3e-7 relative, far inside what the fp16 operands leave of the bar),
            // running pointers, the lo term only when it is stored.
            for (int cb = 16 * part; cb < n; cb += 48) {
                float g[16], u[16], rex[16], rinv[16];
#pragma unroll
                for (int j4 = 0; j4 < 4; j4++) {
                    const float4 r = srex4[(cb >> 2) + j4], ri = saux4[(cb >> 2) + j4];
                    rex[4 * j4] = r.x * sg; rex[4 * j4 + 1] = r.y * sg; rex[4 * j4 + 2] = r.z * sg; rex[4 * j4 + 3] = r.w * sg;
                    rinv[4 * j4] = ri.x * su; rinv[4 * j4 + 1] = ri.y * su; rinv[4 * j4 + 2] = ri.z * su; rinv[4 * j4 + 3] = ri.w * su;
                }
                um_ld16(t0 + cb, g);
                um_ld16(t1 + cb, u);
                if (o < OUT) {
                    __half *ph = Yh + (size_t)(row0 + cb) * OUT + pcol, *pl = Yl + (size_t)(row0 + cb) * OUT + pcol;
                    const int m = min(16, n - cb);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        if (j < m) {
                            // gate at its true size (x 2^e); the up value stays divided by 2^e and the product is divided once more
                            const float gv = g[j] * rex[j];
                            float y = __fdividef(gv, 1.f + __expf(-gv)) * (u[j] * rinv[j]);
                            clamped |= !(fabsf(y) <= 65504.f);
                            y = fminf(fmaxf(y, -65504.f), 65504.f);
                            const __half hi = __float2half_rn(y);
                            ph[(size_t)j * OUT] = hi;
                            if (two_terms) pl[(size_t)j * OUT] = __float2half_rn(y - __half2float(hi));
                        }
                    }
                }
            }
        } else {
            float *Y = reinterpret_cast<float *>(a.Y0);
#pragma unroll
            for (int t = 0; t < 2; t++) {
                const int o = pr * 256 + t * 128 + trow;
                const float sc = o < OUT ? ws[o] : 0.f;
                // (SiLU(gate)*up came in divided by the square of the row's power of two: the slot rows stay divided by it,
                // and the combine step multiplies the token's sum back)
                for (int cb = 16 * part; cb < n; cb += 48) {
                    float v[16];
                    um_ld16((t ? t1 : t0) + cb, v);
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (cb + j < n && o < OUT) Y[(size_t)(row0 + cb + j) * OUT + o] = v[j] * sc;
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) um_bar_arrive(um_s32(&b_acc_free));
        return true;
    };

    if (warp == UM_WARP_TMA) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            unsigned kk = 0;
            for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x) {
                int gi, c0, pr; decode(item, gi, c0, pr);
                const int e = a.gexp[gi] - a.expert_lo, n = min(CR, a.gcnt[gi] - c0), row0 = a.gbeg[gi] + c0;
                const int R = tile_rows(n);
                const CUtensorMap *th = R == 16 ? &tmH16 : R == 32 ? &tmH32 : R == 64 ? &tmH64 : &tmH128;
                const CUtensorMap *tl = R == 16 ? &tmL16 : R == 32 ? &tmL32 : R == 64 ? &tmL64 : &tmL128;
                const int wrow = e * nrows_w + pr * OPP;                 // first weight row of the pair (gate rows for gate/up)
                const unsigned rawA = 2u * UM_RAW_A, bt = (unsigned)R * 128u;
                for (int sl = 0; sl < NST; sl++, kk++) {
                    const unsigned s = kk % STG;
                    if (kk >= STG && !um_bar_wait(um_s32(&b_raw_free[s]), ((kk / STG) - 1) & 1, abortp)) {
                        atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; break;
                    }
                    unsigned char *sp = smem + s * SBYTES;
                    const unsigned bar = um_s32(&b_raw_full[s]);
                    um_bar_expect(bar, rawA + (two_terms ? 4u : 2u) * bt);
                    um_tma_2d(um_s32(sp), &tmW, sl * 64, wrow, bar);                                  // 128 rows x 64 B
                    um_tma_2d(um_s32(sp + rawA / 2), &tmW, sl * 64, wrow + (GATEUP ? OUT : 128), bar);
                    um_tma_2d(um_s32(sp + rawA), th, sl * 128, row0, bar);                             // columns [128 sl, +64)
                    um_tma_2d(um_s32(sp + rawA + bt), th, sl * 128 + 64, row0, bar);                   // columns [128 sl + 64, +64)
                    if (two_terms) {
                        um_tma_2d(um_s32(sp + rawA + 2 * bt), tl, sl * 128, row0, bar);
                        um_tma_2d(um_s32(sp + rawA + 3 * bt), tl, sl * 128 + 64, row0, bar);
                    }
                }
            }
        }
    } else if (warp >= UM_WARP_MMA) {
        // ------------------------------ MMA issuers ------------------------------
        // Two warps: issuer t multiplies tile t of the pair into its own accumulator columns
        // [128 t, 128 t + R).  One MMA of N = R per 16 columns and term: A (the dequantised weights) from tensor
        // memory, B (the fp16 activations) from the slot.
        // The whole warp runs this loop with warp-uniform values; an elected lane issues the MMAs and the commits.
        {
            const int t = __shfl_sync(0xffffffffu, warp, 0) - UM_WARP_MMA;
            const unsigned leader = um_elect();                         // the same lane issues every MMA and every commit
            unsigned ks = 0, nitem = 0;                                  // step and item counters
            for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x, nitem++) {
                int gi, c0, pr; decode(item, gi, c0, pr);
                const int n = __shfl_sync(0xffffffffu, min(CR, a.gcnt[gi] - c0), 0);
                const int R = tile_rows(n);
                const unsigned idesc = (1u << 4) | ((unsigned)(R >> 3) << 17) | ((128u >> 4) << 24);   // f32 accum, f16 x f16, K-major
                const unsigned d_tmem = tmem + (unsigned)t * 128;
                // one accumulator buffer: the previous item's epilogue has to have read it
                if (nitem >= 1 && !um_bar_wait(um_s32(&b_acc_free), (nitem - 1) & 1, abortp)) {
                    if (lane == 0) atomicOr(a.status, SW_ST_TIMEOUT);
                    *abortp = 1; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned bt = (unsigned)R * 128u;
                bool ok = true;
                for (int st = 0; st < NST; st++, ks++) {
                    const unsigned s = ks % STG, kk = 2 * ks + t, b = kk % UM_ABUF;
                    // the dequantising warps announce a tile only after they have seen the slot land (raw rows AND activations)
                    if (!um_bar_wait(um_s32(&b_a_full[b]), (kk / UM_ABUF) & 1, abortp)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned ta = tmem + UM_TMEM_A + b * 64;
                    const unsigned bb = um_s32(smem + s * SBYTES + 2 * UM_RAW_A);
#pragma unroll
                    for (int k = 0; k < 8; k++) {                       // 16 columns per MMA: 8 tensor-memory columns of A, 32 bytes of each B row
                        const uint64_t dh = um_desc(bb + (k >> 2) * bt) + 2 * (k & 3);
                        um_mma_ta_lead(leader, d_tmem, ta + 8 * k, dh, idesc, (st | k) ? 1u : 0u);
                        if (two_terms) um_mma_ta_lead(leader, d_tmem, ta + 8 * k, um_desc(bb + (2 + (k >> 2)) * bt) + 2 * (k & 3), idesc, 1u);
                    }
                    // two commits per step and issuer: the A tile goes back to this tile's dequantising warps (who then do
                    // not wait for the other tile's MMAs), and when both issuers have arrived the slot returns to the TMA warp
                    um_commit_lead(leader, um_s32(&b_a_free[b]));
                    um_commit_lead(leader, um_s32(&b_raw_free[s]));
                }
                if (!ok) { if (lane == 0) atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; break; }
                um_commit_lead(leader, um_s32(&b_acc_full[t]));
            }
        }
    } else if (warp < UM_DQ_WARPS) {
        // ------------------------------ dequantise ------------------------------
        // Two groups of four warps: group t dequantises tile t of every step.  A thread owns one tile row (tensor-memory
        // lane 32 * (warp % 4) + lane): it reads the row's 64 raw bytes of the step from the slot, expands them to 128 exact
        // fp16 integers (nibble - 8) and stores them to the 64 columns of A tile (2 * step + t) % 4 in four pieces.
        // (Sixteen warps with half a row each were slower: 1.02 against 0.96 ms on the 4096-token prefill.  Eight warps
        // stream 146 bytes per clock into tensor memory next to the MMAs, sixteen 186.  A third ring position for chunks
        // of at most 64 rows -- in the accumulators' unused halves, or with the accumulators packed into 128 columns --
        // was slower too, three times out of three: 2.51 against 2.33 ms on the 1024-token very large layer.)
        const int tsel = warp >> 2, q = warp & 3;
        const int trow = q * 32 + lane;
        const unsigned lane_base = (unsigned)(q * 32) << 16;
        unsigned ks = 0, nitem = 0;
        bool clamped = false;
        for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x, nitem++) {
            for (int st = 0; st < NST; st++, ks++) {
                const unsigned kk = 2 * ks + tsel, b = kk % UM_ABUF, s = ks % STG;
                bool ok = um_bar_wait(um_s32(&b_raw_full[s]), (ks / STG) & 1, abortp);
                // A tile b was last read by this tile's MMAs of the step UM_A_SLOTS back: wait until they have retired
                if (ok && ks >= UM_A_SLOTS) ok = um_bar_wait(um_s32(&b_a_free[b]), ((kk / UM_ABUF) - 1) & 1, abortp);
                if (!ok) { if (lane == 0) { atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; } break; }
                // the row's 64 bytes; the TMA wrote them under the 64-byte swizzle: 16-byte chunk c sits at c ^ ((row >> 1) & 3)
                const unsigned char *rrow = smem + s * SBYTES + (size_t)(tsel * 128 + trow) * 64;
                const int sw = (trow >> 1) & 3;
                uint4 wv[4];
#pragma unroll
                for (int c = 0; c < 4; c++) wv[c] = *reinterpret_cast<const uint4 *>(rrow + ((c ^ sw) << 4));
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int qt = 0; qt < 4; qt++) {                        // four independent quarters (32 fp16 = 16 columns each): a
                    uint32_t r[16];                                     // quarter's store drains while the next one is converted
                    const uint32_t ww[4] = {wv[qt].x, wv[qt].y, wv[qt].z, wv[qt].w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {                       // word i: columns 8i .. 8i+7 in the order 0,4,1,5,2,6,3,7
                        const uint4 d = um_dq(ww[i]);
                        r[4 * i] = d.x; r[4 * i + 1] = d.y; r[4 * i + 2] = d.z; r[4 * i + 3] = d.w;
                    }
                    um_st16_nowait(tmem + lane_base + UM_TMEM_A + b * 64 + qt * 16, r);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) um_bar_arrive(um_s32(&b_a_full[b]));
            }
            if (*abortp) break;
            // this item's tiles are all handed over: help with its epilogue (nothing can be dequantised into the A ring
            // until the MMAs that read it have retired, and those are the ones the accumulators are waiting for)
            if (!epilogue_share(item, nitem, 1 + tsel, clamped)) break;
        }
        if (clamped) atomicOr(a.status, SW_ST_RANGE);
    } else {
        // ------------------------------ epilogue warps (one TMEM lane quarter each; share 0 of 3) ------------------------------
        unsigned nitem = 0;
        bool clamped = false;
        for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x, nitem++) {
            if (GATEUP) {   // this item's per-row powers of two -> shared memory (128 entries, ones past the chunk's end)
                int gi, c0, pr; decode(item, gi, c0, pr);
                const int n = min(CR, a.gcnt[gi] - c0), row0 = a.gbeg[gi] + c0, i = (warp - UM_DQ_WARPS) * 32 + lane;
                const float r = (a.srex && i < n) ? a.srex[row0 + i] : 1.f;
                s_srex[nitem & 1][0][i] = r;
                s_srex[nitem & 1][1][i] = __frcp_rn(r);
                __syncwarp();
                if (lane == 0) um_bar_arrive(um_s32(&b_srex[nitem & 1]));
            }
            if (!epilogue_share(item, nitem, 0, clamped)) break;
        }
        if (clamped) atomicOr(a.status, SW_ST_RANGE);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == UM_WARP_MMA) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512) : "memory");
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*um_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static um_encode_fn um_get_encode() {
    // looked up once (thread-safe static initialisation); NULL when the driver does not export the encoder
    static const um_encode_fn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            return (um_encode_fn)p;
        cudaGetLastError();
        return (um_encode_fn)nullptr;
    }();
    return fn;
}
static int um_make_map(CUtensorMap *m, CUtensorMapDataType dt, int esize, const void *ptr, long long inner, long long rows,
                       int box_inner, int box_rows, CUtensorMapSwizzle sw) {
    um_encode_fn enc = um_get_encode();
    if (!enc) return -1;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)inner * esize};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, dt, 2, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -1;
}

bool sw_umma_available() { return um_get_encode() != nullptr; }

int sw_launch_row_exp(const SwLaunchCfg &c, const float *x, int rows, int KD, float *rexp) {
    if (rows <= 0) return 0;
    if (KD % 4) return -1;
    int grid = (rows + 7) / 8;
    if (grid > c.num_sms * 8) grid = c.num_sms * 8;
    k_row_exp<<<grid, 256, 0, c.stream>>>(x, rows, KD, rexp);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// rexp / srex (both or neither): rexp[token row] = the power of two to divide the row by, srex[packed row] receives a copy
int sw_launch_umma_gather(const SwLaunchCfg &c, const float *x, const int *grow, const int *npairs, int P, int KD, void *hi, void *lo, int *status,
                          const float *rexp, float *srex) {
    if (P <= 0) return 0;
    if ((rexp == nullptr) != (srex == nullptr)) return -1;
    long long grid = ((long long)P + 7) / 8;                            // a warp per packed row, eight warps per CTA
    if (grid > (long long)c.num_sms * 16) grid = (long long)c.num_sms * 16;
    k_umma_gather<<<(unsigned)grid, 256, 0, c.stream>>>(x, grow, npairs, P, KD, (__half *)hi, (__half *)lo, status, rexp, srex);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int sw_umma_chunk_rows(bool small) { return small ? 32 : 128; }

int sw_launch_umma_chunks(const SwLaunchCfg &c, const SwQ4Args &a, int *nchunks, void *chunks, bool small) {
    k_umma_chunks<<<1, 1024, 0, c.stream>>>(a.G, a.gexp, a.gcnt, a.expert_lo, a.expert_cnt, nchunks, (int2 *)chunks, sw_umma_chunk_rows(small));
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// act_hi/act_lo: fp16 [max_rows, KD] in packed-slot order (permuted columns).
// gate/up: Y0/Y1 = fp16 hi/lo [max_rows, OUT]; down: Y0 = f32 [max_rows, OUT].
int sw_launch_q4_umma(const SwLaunchCfg &c, const SwQ4Args &a, const void *act_hi, const void *act_lo, void *Y0, void *Y1,
                      const int *nchunks, const void *chunks, int max_chunks, int *status, long long wrows_total, bool gateup, int terms,
                      const float *srex, bool small) {
    if (a.max_rows <= 0) return 0;
    if (terms != 1 && terms != 2) return -1;
    if (terms == 1) act_lo = act_hi;                                    // never read; keeps the tensor maps valid
    if (a.KD % 128 || a.OUT <= 0 || ((uintptr_t)a.q & 15)) return -1;
    if ((a.OUT % (gateup ? 128 : 256)) != 0) return -1;                  // whole tile pairs only
    CUtensorMap tw, th[4], tl[4];
    if (um_make_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.q, a.KD / 2, wrows_total, 64, 128, CU_TENSOR_MAP_SWIZZLE_64B)) return -1;
    const int R[4] = {16, 32, 64, 128};
    for (int i = 0; i < 4; i++) {
        if (um_make_map(&th[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, act_hi, a.KD, a.max_rows, 64, R[i], CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
        if (um_make_map(&tl[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, act_lo, a.KD, a.max_rows, 64, R[i], CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    }
    static_assert(UM_STAGES_FOR(1) * UM_STAGE_BYTES(1) <= UM_RING_BYTES && UM_STAGES_FOR(2) * UM_STAGE_BYTES(2) <= UM_RING_BYTES, "ring sizes");
    static_assert(UM_A_SLOTS <= UM_STAGES_FOR(1) && UM_A_SLOTS <= UM_STAGES_FOR(2), "an A tile's release is read off the slot barrier of its step");
    constexpr int SMEM = UM_RING_BYTES + 1024;
    static SwPerDevice attr;
    if (attr.get(c.dev, [] {
            if (cudaFuncSetAttribute(k_q4_umma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
                cudaFuncSetAttribute(k_q4_umma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    UmArgs ka;
    ka.Ws = a.s; ka.Y0 = Y0; ka.Y1 = Y1; ka.gexp = a.gexp; ka.gbeg = a.gbeg; ka.gcnt = a.gcnt; ka.nchunks = nchunks;
    ka.chunks = (const int2 *)chunks; ka.status = status; ka.KD = a.KD; ka.OUT = a.OUT; ka.expert_lo = a.expert_lo; ka.terms = terms; ka.srex = srex;
    ka.chunk_rows = sw_umma_chunk_rows(small);
    if (small) { ka.stage_bytes = 2 * UM_RAW_A + 2 * terms * (32 * 128); ka.stages = UM_RING_BYTES / ka.stage_bytes; if (ka.stages > UM_MAX_STAGES) ka.stages = UM_MAX_STAGES; }
    else { ka.stage_bytes = UM_STAGE_BYTES(terms); ka.stages = UM_STAGES_FOR(terms); }
    const int pairs = a.OUT / (gateup ? 128 : 256);
    long long items = (long long)max_chunks * pairs;
    long long grid = c.num_sms;                        // one CTA per SM (shared memory and tensor memory are sized for that)
    if (grid > items) grid = items;
    if (grid < 1) grid = 1;
    if (gateup) k_q4_umma<true><<<(unsigned)grid, UM_THREADS, SMEM, c.stream>>>(tw, th[0], th[1], th[2], th[3], tl[0], tl[1], tl[2], tl[3], ka);
    else k_q4_umma<false><<<(unsigned)grid, UM_THREADS, SMEM, c.stream>>>(tw, th[0], th[1], th[2], th[3], tl[0], tl[1], tl[2], tl[3], ka);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ===========================================================================
// Dense bf16 shared expert on tcgen05 for many token rows (prefill).
// Same pipeline without the dequantise stage: the bf16 weight tile arrives by TMA
// already in the layout the tensor core reads (64 columns x 128 rows, 128B
// swizzle); the activations are two bf16 terms (x = hi + lo) in planar [T, K]
// arrays.  Gate rows fill tile rows 0..63 and up rows 64..127, so the epilogue
// warps of the upper half hand their values to the lower half through shared
// memory.  Work item = (m-tile, chunk of 128 token rows).
// ===========================================================================
#define UB_STAGES 4
#define UB_STAGE_BYTES (3 * UM_BT)
#define UB_THREADS (6 * 32)

__global__ void __launch_bounds__(256)
k_pack_bf16_planar(const float *__restrict__ x, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, size_t n8) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n8; idx += (size_t)gridDim.x * blockDim.x) {
        const float4 *src = reinterpret_cast<const float4 *>(x) + idx * 2;
        const float4 a = src[0], b = src[1];
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        __nv_bfloat16 h[8], l[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { h[i] = __float2bfloat16_rn(v[i]); l[i] = __float2bfloat16_rn(v[i] - __bfloat162float(h[i])); }
        reinterpret_cast<uint4 *>(hi)[idx] = *reinterpret_cast<uint4 *>(h);
        reinterpret_cast<uint4 *>(lo)[idx] = *reinterpret_cast<uint4 *>(l);
    }
}

struct UbArgs { void *Y0, *Y1; int T, KD, O; int *status; };

template <bool GATEUP>
__global__ void __launch_bounds__(UB_THREADS, 1)
k_bf16_umma(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
            const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmL, const UbArgs a) {
    extern __shared__ unsigned char um_dyn[];
    __shared__ unsigned long long b_full[UB_STAGES], b_free[UB_STAGES], b_acc_full[2], b_acc_free[2];
    __shared__ unsigned s_tmem;
    __shared__ int s_abort;
    __shared__ float s_ex[64][33];                                       // up values of one 32-column block
    unsigned char *smem = (unsigned char *)(((uintptr_t)um_dyn + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = a.T, KD = a.KD, O = a.O;
    constexpr int OPT = GATEUP ? 64 : 128;
    const int mtiles = (O + OPT - 1) / OPT, chunks = (T + 127) >> 7;
    const int items = mtiles * chunks;
    const int NST = KD >> 6;
    volatile int *abortp = &s_abort;

    if (threadIdx.x == 0) {
        for (int i = 0; i < UB_STAGES; i++) { um_bar_init(um_s32(&b_full[i]), 1); um_bar_init(um_s32(&b_free[i]), 1); }
        for (int i = 0; i < 2; i++) { um_bar_init(um_s32(&b_acc_full[i]), 1); um_bar_init(um_s32(&b_acc_free[i]), 4); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(um_s32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = s_tmem;

    if (warp == 4) {
        if (lane == 0) {                                                 // TMA producer
            unsigned kk = 0;
            for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x) {
                const int ci = item / mtiles, mt = item - ci * mtiles;   // m-tiles of one chunk are neighbours: the chunk stays in L2
                for (int st = 0; st < NST; st++, kk++) {
                    const int s = kk % UB_STAGES;
                    if (kk >= UB_STAGES && !um_bar_wait(um_s32(&b_free[s]), ((kk / UB_STAGES) - 1) & 1, abortp)) {
                        atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; break;
                    }
                    unsigned char *sp = smem + s * UB_STAGE_BYTES;
                    const unsigned bar = um_s32(&b_full[s]);
                    um_bar_expect(bar, 3u * UM_BT);
                    if (GATEUP) {
                        um_tma_2d(um_s32(sp), &tmW0, st * 64, mt * 64, bar);
                        um_tma_2d(um_s32(sp + UM_BT / 2), &tmW1, st * 64, mt * 64, bar);
                    } else {
                        um_tma_2d(um_s32(sp), &tmW0, st * 64, mt * 128, bar);
                    }
                    um_tma_2d(um_s32(sp + UM_BT), &tmH, st * 64, ci * 128, bar);
                    um_tma_2d(um_s32(sp + 2 * UM_BT), &tmL, st * 64, ci * 128, bar);
                }
            }
        }
    } else if (warp == 5) {
        {                                                                // MMA issuer: the whole warp, warp-uniform; an elected lane issues
            unsigned kk = 0, tile = 0;
            for (int item = blockIdx.x; item < items && !*abortp; item += gridDim.x, tile++) {
                const int ci = item / mtiles;
                // hi and lo tiles are adjacent: one N=256 MMA per step, columns [0,128) = A*hi, [128,256) = A*lo
                const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);  // f32 accum, bf16 x bf16
                const unsigned acc = tile & 1, d_tmem = tmem + acc * 256;
                if (tile >= 2 && !um_bar_wait(um_s32(&b_acc_free[acc]), ((tile >> 1) - 1) & 1, abortp)) { if (lane == 0) atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int st = 0; st < NST; st++, kk++) {
                    const int s = kk % UB_STAGES;
                    if (!um_bar_wait(um_s32(&b_full[s]), (kk / UB_STAGES) & 1, abortp)) { if (lane == 0) atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned char *sp = smem + s * UB_STAGE_BYTES;
                    const uint64_t da = um_desc(um_s32(sp)), db = um_desc(um_s32(sp + UM_BT));
#pragma unroll
                    for (int k = 0; k < 4; k++) um_mma_elect(d_tmem, da + 2 * k, db + 2 * k, idesc, (st | k) ? 1u : 0u);
                    um_commit_elect(um_s32(&b_free[s]));
                }
                if (*abortp) break;
                um_commit_elect(um_s32(&b_acc_full[acc]));
            }
        }
    } else {
        // epilogue warps 0-3: warp q owns accumulator rows 32q..32q+31
        const int q = warp, trow = q * 32 + lane;
        unsigned tile = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, tile++) {
            const int ci = item / mtiles, mt = item - ci * mtiles;
            const int n = min(128, T - ci * 128), row0 = ci * 128;
            const unsigned acc = tile & 1;
            bool ok = !*abortp && um_bar_wait(um_s32(&b_acc_full[acc]), (tile >> 1) & 1, abortp);
            if (!ok && lane == 0) { atomicOr(a.status, SW_ST_TIMEOUT); *abortp = 1; }
            // the four warps stay in step through the named barrier even on an abort
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int cb = 0; cb < 128; cb += 32) {
                float v[32];
                if (ok && cb < n) {
                    float p[32];
                    um_ld32(tmem + acc * 256 + cb + ((unsigned)(q * 32) << 16), v);
                    um_ld32(tmem + acc * 256 + 128 + cb + ((unsigned)(q * 32) << 16), p);
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] += p[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = 0.f;
                }
                if (GATEUP) {
                    if (q >= 2) {
#pragma unroll
                        for (int j = 0; j < 32; j++) s_ex[trow - 64][j] = v[j];
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (q < 2 && ok) {
                        const int o = mt * 64 + trow;
                        __nv_bfloat16 *Yh = reinterpret_cast<__nv_bfloat16 *>(a.Y0), *Yl = reinterpret_cast<__nv_bfloat16 *>(a.Y1);
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            if (cb + j < n && o < O) {
                                const float gv = v[j], uv = s_ex[trow][j];
                                const float y = (gv / (1.f + expf(-gv))) * uv;
                                const __nv_bfloat16 hi = __float2bfloat16_rn(y), lo = __float2bfloat16_rn(y - __bfloat162float(hi));
                                const size_t pos = (size_t)(row0 + cb + j) * O + o;
                                Yh[pos] = hi; Yl[pos] = lo;
                            }
                        }
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                } else if (ok) {
                    float *Y = reinterpret_cast<float *>(a.Y0);
                    const int o = mt * 128 + trow;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (cb + j < n && o < O) Y[(size_t)(row0 + cb + j) * O + o] = v[j];
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) um_bar_arrive(um_s32(&b_acc_free[acc]));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512) : "memory");
    }
}

int sw_launch_pack_bf16_planar(const SwLaunchCfg &c, const float *x, void *hi, void *lo, int rows, int KD) {
    if (rows <= 0) return 0;
    if (KD % 8) return -1;
    size_t n8 = (size_t)rows * (KD / 8);
    long long grid = (long long)((n8 + 255) / 256);
    if (grid > (long long)c.num_sms * 16) grid = (long long)c.num_sms * 16;
    k_pack_bf16_planar<<<(unsigned)grid, 256, 0, c.stream>>>(x, (__nv_bfloat16 *)hi, (__nv_bfloat16 *)lo, n8);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// W0 (and W1 for gate/up): bf16 [O, KD]; act_hi/lo: bf16 [T, KD]; gate/up -> Y0/Y1 bf16 hi/lo [T, O]; down -> Y0 f32 [T, O]
int sw_launch_bf16_umma(const SwLaunchCfg &c, const void *W0, const void *W1, const void *act_hi, const void *act_lo,
                        void *Y0, void *Y1, int T, int KD, int O, int *status, bool gateup) {
    if (T <= 0 || O <= 0) return 0;
    if (KD % 64 || (((uintptr_t)W0 | (uintptr_t)(W1 ? W1 : W0)) & 15)) return -1;
    CUtensorMap tw0, tw1, th, tl;
    const int wrows = gateup ? 64 : 128;
    if (um_make_map(&tw0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W0, KD, O, 64, wrows, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (um_make_map(&tw1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, gateup ? W1 : W0, KD, O, 64, wrows, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (um_make_map(&th, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, act_hi, KD, T, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    if (um_make_map(&tl, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, act_lo, KD, T, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return -1;
    constexpr int SMEM = UB_STAGES * UB_STAGE_BYTES + 1024;
    static SwPerDevice attr;
    if (attr.get(c.dev, [] {
            if (cudaFuncSetAttribute(k_bf16_umma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
                cudaFuncSetAttribute(k_bf16_umma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    UbArgs ka{Y0, Y1, T, KD, O, status};
    const int opt = gateup ? 64 : 128;
    long long items = (long long)((O + opt - 1) / opt) * ((T + 127) / 128);
    long long grid = c.num_sms < items ? c.num_sms : items;
    if (gateup) k_bf16_umma<true><<<(unsigned)grid, UB_THREADS, SMEM, c.stream>>>(tw0, tw1, th, tl, ka);
    else k_bf16_umma<false><<<(unsigned)grid, UB_THREADS, SMEM, c.stream>>>(tw0, tw1, th, tl, ka);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
