// Router logits, gate activation + top-k, and the device-side group-by-expert
// dispatch (histogram, prefix scan, stable permute) of the MoE block.
//
// Reference behaviour restated here:
//   router logits   c/laguna.c:574-576,698 (matmul_f32; exact contract c/moe_matmul.h:46-54)
//   gate            c/moe_block.h:25-26, softmax_row c/moe_math.h:68-72, softplusf c/moe_math.h:54
//   top-k           moe_topk, c/moe_arch.h:64-89
//   weights         c/moe_block.h:30-31, c/laguna.c:704-705
//   dispatch        counting sort, c/laguna.c:709-723
#include "sw_common.cuh"

// ---------------------------------------------------------------------------
// Router logits: rl[t,e] = (float) sum_k (double)x[t,k]*W[e,k]  (+ logit_bias[e]).
// One warp per expert row, TT tokens per pass, fp64 accumulation: the product of
// two f32 is exact in fp64, so only the order of the additions differs from the
// reference's sequential double sum, and the result is rounded to f32 once.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void sw_load8(const float *p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void sw_load8(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4 *>(p);
    uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i]     = __uint_as_float(u[i] << 16);
        v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

template <typename WT, int TT>
__global__ void __launch_bounds__(256)
k_router_logits(const float *__restrict__ x, const WT *__restrict__ W, const float *__restrict__ lbias,
                float *__restrict__ rl, int T, int D, int E) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * TT;
    if (e >= E) return;
    double acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.0;
    const WT *wr = W + (size_t)e * D;
    for (int k = lane * 8; k < D; k += 256) {
        float wv[8];
        sw_load8(wr + k, wv);
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (t0 + t < T) {
                float xv[8];
                sw_load8(x + (size_t)(t0 + t) * D + k, xv);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[t] = fma((double)xv[i], (double)wv[i], acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        double a = acc[t];
#pragma unroll
        for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(SW_FULL_MASK, a, off);
        if (lane == 0 && t0 + t < T) {
            float r = (float)a;
            if (lbias) r += lbias[e];
            rl[(size_t)(t0 + t) * E + e] = r;
        }
    }
}

int sw_launch_router_logits(const SwLaunchCfg &c, const float *x, const void *W, int w_dtype,
                            const float *logit_bias, float *rl, int T, int D, int E) {
    if (T <= 0) return 0;
    if (D % 8) return -1;
    constexpr int TT = 4;
    dim3 grid((E + 7) / 8, (T + TT - 1) / TT);
    if (w_dtype == 1)
        k_router_logits<__nv_bfloat16, TT><<<grid, 256, 0, c.stream>>>(x, (const __nv_bfloat16 *)W, logit_bias, rl, T, D, E);
    else
        k_router_logits<float, TT><<<grid, 256, 0, c.stream>>>(x, (const float *)W, logit_bias, rl, T, D, E);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// Router logits on the fp64 tensor cores (mma.sync m8n8k4 f64).  Warp item =
// (tile of 8 experts, pass of up to 32 token rows, slice of 256 columns); the
// slices' partial sums go to part[slice][t][e] in fp64 and are added in a fixed
// order by the top-k kernel before the single rounding to f32.  Lane (r, c) feeds
// the k-slot c of step j with column 8c+j of the 32-column step, so both the
// weight row (16 bytes of bf16 / 32 of f32) and the token row (32 bytes) are
// contiguous loads.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void sw_dmma(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c[0]), "+d"(c[1]) : "d"(a), "d"(b));
}

// NT = token n-tiles (of 8 rows) per warp item: 4 for large batches (weights re-used across 32 rows), 1 for
// small batches, where more, shorter warp items hide the latency of the dependent fp64 MMA chains.
template <typename WT, int NT>
__global__ void __launch_bounds__(128)
k_router_dmma(const float *__restrict__ x, const WT *__restrict__ W, double *__restrict__ part,
              int T, int D, int E, int KS, int slice) {
    const int lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3;
    const int warps_total = gridDim.x * 4, wid = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int etiles = (E + 7) >> 3, passes = (T + 8 * NT - 1) / (8 * NT);
    const int items = etiles * passes * KS;
    for (int item = wid; item < items; item += warps_total) {
        const int ks = item % KS, rest = item / KS, et = rest % etiles, ps = rest / etiles;
        const int k0 = ks * slice, k1 = min(D, k0 + slice);
        const int e = min(et * 8 + r, E - 1);
        const WT *wr = W + (size_t)e * D + c * 8;
        const float *xr[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) xr[nt] = x + (size_t)min(ps * 8 * NT + nt * 8 + r, T - 1) * D + c * 8;
        const int nt_used = min(NT, (T - ps * 8 * NT + 7) >> 3);
        double acc[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { acc[nt][0] = 0.0; acc[nt][1] = 0.0; }
        for (int k = k0; k < k1; k += 32) {
            float wv[8];
            sw_load8(wr + k, wv);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                if (nt < nt_used) {
                    float xv[8];
                    sw_load8(xr[nt] + k, xv);
#pragma unroll
                    for (int j = 0; j < 8; j++) sw_dmma(acc[nt], (double)wv[j], (double)xv[j]);
                }
            }
        }
        // C[row = expert r][col = token 2c, 2c+1]
        const int eo = et * 8 + r;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            if (nt >= nt_used || eo >= E) continue;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int t = ps * 8 * NT + nt * 8 + 2 * c + j;
                if (t < T) part[((size_t)ks * T + t) * E + eo] = acc[nt][j];
            }
        }
    }
}

// The same product for many token rows (prefill, large batches): a CTA computes a tile of 64 experts x 64 token rows
// from operands staged in shared memory AS DOUBLES, 32 columns per stage, two stages.  The kernel above streams its
// operands from L2 into registers for every 8 x 32 tile (3.6 flop per byte: at 4096 tokens it moves 5.8 TB/s out of L2
// and runs at half the fp64 tensor rate) and converts every value once per use; here a value is loaded and converted
// once per 64 x 64 tile.  Eight warps, each 16 experts x 32 tokens = 2 x 4 MMA tiles.  Rows are padded to 36 doubles:
// the 16 lanes of a half-warp (4 rows x 4 k-slots) then read 32 different banks.
#define RT_TILE 64
#define RT_LD 36
#define RT_SMEM (2 * 2 * RT_TILE * RT_LD * 8)
template <typename WT>
__global__ void __launch_bounds__(256)
k_router_dmma_tiled(const float *__restrict__ x, const WT *__restrict__ W, double *__restrict__ part,
                    int T, int D, int E, int KS, int slice) {
    extern __shared__ __align__(16) unsigned char rt_dyn[];
    double (*sm)[2][RT_TILE][RT_LD] = reinterpret_cast<double (*)[2][RT_TILE][RT_LD]>(rt_dyn);   // [buffer][A|B][row][col]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, c = lane & 3;
    const int etiles = (E + RT_TILE - 1) / RT_TILE, ttiles = (T + RT_TILE - 1) / RT_TILE;
    const int items = etiles * ttiles * KS;
    const int frow = tid >> 2, fcol = (tid & 3) * 8;          // this thread's row and first column when filling a stage
    const int m0 = (warp & 3) * 16, n0 = (warp >> 2) * 32;    // this warp's experts and tokens inside the tile
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        // the expert tiles of one (token tile, slice) are neighbours: the token rows stay in L2
        const int et = item % etiles, rest = item / etiles, ks = rest % KS, tt = rest / KS;
        const int k0 = ks * slice, k1 = min(D, k0 + slice);
        const int e0 = et * RT_TILE, t0 = tt * RT_TILE;
        const WT *wr = W + (size_t)min(e0 + frow, E - 1) * D + fcol;
        const float *xr = x + (size_t)min(t0 + frow, T - 1) * D + fcol;
        double acc[2][4][2];
#pragma unroll
        for (int mi = 0; mi < 2; mi++)
#pragma unroll
            for (int ni = 0; ni < 4; ni++) { acc[mi][ni][0] = 0.0; acc[mi][ni][1] = 0.0; }
        float wv[8], xv[8];
        if (k0 < k1) { sw_load8(wr + k0, wv); sw_load8(xr + k0, xv); }
        __syncthreads();                                       // the previous item's last stage has been read
        for (int k = k0, st = 0; k < k1; k += 32, st++) {
            double (*A)[RT_LD] = sm[st & 1][0], (*B)[RT_LD] = sm[st & 1][1];
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                *reinterpret_cast<double2 *>(&A[frow][fcol + i]) = make_double2((double)wv[i], (double)wv[i + 1]);
                *reinterpret_cast<double2 *>(&B[frow][fcol + i]) = make_double2((double)xv[i], (double)xv[i + 1]);
            }
            __syncthreads();
            if (k + 32 < k1) { sw_load8(wr + k + 32, wv); sw_load8(xr + k + 32, xv); }   // in flight under the MMAs
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                double a[2], b[4];
#pragma unroll
                for (int mi = 0; mi < 2; mi++) a[mi] = A[m0 + mi * 8 + r][4 * kk + c];
#pragma unroll
                for (int ni = 0; ni < 4; ni++) b[ni] = B[n0 + ni * 8 + r][4 * kk + c];
#pragma unroll
                for (int mi = 0; mi < 2; mi++)
#pragma unroll
                    for (int ni = 0; ni < 4; ni++) sw_dmma(acc[mi][ni], a[mi], b[ni]);
            }
            // the stage after next overwrites this buffer; every warp passes the barrier above (of the next stage) first
        }
        // C[row = expert r][col = token 2c, 2c+1] of every MMA tile
#pragma unroll
        for (int mi = 0; mi < 2; mi++) {
            const int eo = e0 + m0 + mi * 8 + r;
            if (eo >= E) continue;
#pragma unroll
            for (int ni = 0; ni < 4; ni++)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int t = t0 + n0 + ni * 8 + 2 * c + j;
                    if (t < T) part[((size_t)ks * T + t) * E + eo] = acc[mi][ni][j];
                }
        }
    }
}

// Token rows from which the tiled kernel is used
#define SW_ROUTER_TILED_MIN_T 128

// Number of column slices the DMMA router uses for (T, E, D); the top-k kernel sums this many partials.
int sw_router_slices(int num_sms, int T, int D, int E) {
    if (T >= SW_ROUTER_TILED_MIN_T) {
        // two CTA items per SM; never finer than 256 columns.  KS * T stays below num_sms * 8192 / E + T, the same bound
        // as for the streaming kernel below, which is what the partial-sum buffer is sized for.
        const int tiles = ((E + RT_TILE - 1) / RT_TILE) * ((T + RT_TILE - 1) / RT_TILE);
        const int want = (num_sms * 2 + tiles - 1) / tiles, maxs = (D + 255) / 256;
        return want < 1 ? 1 : want > maxs ? maxs : want;
    }
    const int nt = T <= 64 ? 1 : 4;
    const int etiles = (E + 7) / 8, passes = (T + 8 * nt - 1) / (8 * nt);
    int want = (num_sms * 32 + etiles * passes - 1) / (etiles * passes);
    int maxs = (D + 127) / 128;
    if (nt == 4 && maxs > (D + 255) / 256) maxs = (D + 255) / 256;
    return want < 1 ? 1 : want > maxs ? maxs : want;
}

int sw_launch_router_dmma(const SwLaunchCfg &c, const float *x, const void *W, int w_dtype, double *part,
                          int T, int D, int E, int KS) {
    if (T <= 0) return 0;
    if (D % 32) return -1;
    int slice = ((D + KS - 1) / KS + 31) & ~31;
    if (T >= SW_ROUTER_TILED_MIN_T) {
        static SwPerDevice attr;
        if (attr.get(c.dev, [] {
                if (cudaFuncSetAttribute(k_router_dmma_tiled<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM) != cudaSuccess ||
                    cudaFuncSetAttribute(k_router_dmma_tiled<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
                return 1; }) <= 0) return -1;
        const long long items = (long long)((E + RT_TILE - 1) / RT_TILE) * ((T + RT_TILE - 1) / RT_TILE) * KS;
        long long grid = (long long)c.num_sms * 2;
        if (grid > items) grid = items;
        if (w_dtype == 1) k_router_dmma_tiled<__nv_bfloat16><<<(unsigned)grid, 256, RT_SMEM, c.stream>>>(x, (const __nv_bfloat16 *)W, part, T, D, E, KS, slice);
        else k_router_dmma_tiled<float><<<(unsigned)grid, 256, RT_SMEM, c.stream>>>(x, (const float *)W, part, T, D, E, KS, slice);
        sw_count_launch();
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }
    const int nt = T <= 64 ? 1 : 4;
    const int etiles = (E + 7) / 8, passes = (T + 8 * nt - 1) / (8 * nt);
    long long items = (long long)etiles * passes * KS, need = (items + 3) / 4;
    long long grid = (long long)c.num_sms * 8;
    if (grid > need) grid = need;
    if (w_dtype == 1) {
        if (nt == 1) k_router_dmma<__nv_bfloat16, 1><<<(unsigned)grid, 128, 0, c.stream>>>(x, (const __nv_bfloat16 *)W, part, T, D, E, KS, slice);
        else k_router_dmma<__nv_bfloat16, 4><<<(unsigned)grid, 128, 0, c.stream>>>(x, (const __nv_bfloat16 *)W, part, T, D, E, KS, slice);
    } else {
        if (nt == 1) k_router_dmma<float, 1><<<(unsigned)grid, 128, 0, c.stream>>>(x, (const float *)W, part, T, D, E, KS, slice);
        else k_router_dmma<float, 4><<<(unsigned)grid, 128, 0, c.stream>>>(x, (const float *)W, part, T, D, E, KS, slice);
    }
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// Dispatch: stable counting sort of the T*K (row, expert) pairs by expert, done
// by ONE CTA of NTH threads.  Each warp owns a contiguous segment of the flat
// pair index, so a per-warp histogram followed by an exclusive scan over
// (expert, warp) gives every warp the first slot of its pairs for each expert;
// walking the segment in order with __match_any ranks keeps pairs of one expert
// in ascending flat index -- the reference's order (c/laguna.c:709-723).
// sm: (NTH/32 + 2) * E ints of shared memory.
// ---------------------------------------------------------------------------
template <int NTH>
__device__ __forceinline__ void sw_dispatch_block(int *sm, const int *sel, int npairs, int K, int E, int T,
                                                  int *Gout, int *gexp, int *gbeg, int *gcnt, int *grow, int *rowof, int *status) {
    constexpr int NW = NTH / 32;
    int *wh = sm;                    // [NW][E] per-warp histogram -> per-warp running slot offset
    int *pos = sm + NW * E;          // [E] first slot of expert e
    int *cnt = pos + E;              // [E]
    __shared__ int s_wsum[32], s_gsum[32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int i = tid; i < NW * E; i += NTH) wh[i] = 0;
    __syncthreads();

    int seg = (npairs + NW - 1) / NW;
    seg = (seg + 31) & ~31;
    const int s0 = min(warp * seg, npairs), s1 = min(s0 + seg, npairs);
    for (int i = s0 + lane; i < s1; i += 32) {
        int e = __ldcg(sel + i);
        if (e == SW_NO_EXPERT) continue;                       // a pair that contributes nothing (rows routed elsewhere)
        if (e < 0 || e >= E) { atomicOr(status, SW_ST_BAD_EXPERT); continue; }
        atomicAdd(&wh[warp * E + e], 1);
    }
    __syncthreads();

    // per expert: total and exclusive prefix over warps
    for (int e = tid; e < E; e += NTH) {
        int run = 0;
        for (int wv = 0; wv < NW; wv++) { int c = wh[wv * E + e]; wh[wv * E + e] = run; run += c; }
        cnt[e] = run;
    }
    __syncthreads();

    // exclusive scan over experts of cnt (slots) and of cnt>0 (group index): every thread owns a run of CH experts
    const int CH = (E + NTH - 1) / NTH;
    const int e0 = tid * CH, e1 = min(E, e0 + CH);
    int c = 0, nz = 0;
    for (int e = e0; e < e1; e++) { c += cnt[e]; nz += cnt[e] > 0 ? 1 : 0; }
    int sc = c, sg = nz;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        int a = __shfl_up_sync(SW_FULL_MASK, sc, off), b = __shfl_up_sync(SW_FULL_MASK, sg, off);
        if (lane >= off) { sc += a; sg += b; }
    }
    if (lane == 31) { s_wsum[warp] = sc; s_gsum[warp] = sg; }
    __syncthreads();
    {
        // every thread adds up the totals of the warps before its own (at most NW - 1 shared-memory reads): one barrier
        // and one single-warp phase less than a second-level scan
        int wbase = 0, gbase = 0;
        for (int wv = 0; wv < warp; wv++) { wbase += s_wsum[wv]; gbase += s_gsum[wv]; }
        int excl = wbase + sc - c, gidx = gbase + sg - nz;
        for (int e = e0; e < e1; e++) {
            const int ce = cnt[e];
            pos[e] = excl;
            if (ce > 0) { gexp[gidx] = e; gbeg[gidx] = excl; gcnt[gidx] = ce; gidx++; }
            excl += ce;
        }
        if (tid == NTH - 1) { Gout[0] = gidx; Gout[1] = excl; }   // groups, and pairs that selected an expert
    }
    __syncthreads();

    // stable scatter
    for (int base = s0; base < s1; base += 32) {
        int i = base + lane;
        int e = i < s1 ? __ldcg(sel + i) : -1;
        bool ok = e >= 0 && e < E;
        unsigned peers = __match_any_sync(SW_FULL_MASK, ok ? e : -1 - lane);
        int off = ok ? wh[warp * E + e] : 0;
        __syncwarp();
        if (ok) {
            int rank = __popc(peers & ((1u << lane) - 1));
            int slot = pos[e] + off + rank;
            int row = i / K;
            if (row >= T) atomicOr(status, SW_ST_BAD_ROW);
            else { grow[slot] = row; rowof[i] = slot; }
            if (rank == 0) wh[warp * E + e] = off + __popc(peers);
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------
// Gate activation + top-k + combine weights: one warp per token.
// exp/log1p are evaluated in fp64 and rounded to f32, which reproduces a
// correctly rounded expf; every other operation is the reference's f32 sequence.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float sw_expf_cr(float v) { return (float)exp((double)v); }

// K selection rounds by one warp (the reference's moe_topk, c/moe_arch.h:64-89): arg-max of score+bias with strict >
// from -1e30f, ties to the lower id, an expert is taken once; if nothing compares greater (all NaN or <= -1e30f) the
// lowest id not yet taken.  Lane l keeps the values of experts l, l+32, ... in registers; a round is a local scan, a
// warp max over an order-preserving integer key and a warp min over the ids that hold that maximum.
// pool (optional): the shared expert shares the routed weight pool (the reference's MOE_SHARED_GATED policy,
// c/inkling.c:1038-1043): weights are the gate scores of the K picks and of the shared expert (s_sc[E]), normalised
// to sum 1 over all K + 1 (float sum: the picks in rank order, then the shared one) and multiplied by pool_scale;
// the shared expert's weight goes to *gate_t.
template <int NJ>
__device__ __forceinline__ void sw_topk_warp(const float *s_sb, const float *s_sc, int E, int K, int norm_topk,
                                             int *sel_t, float *w_t, bool pool = false, float pool_scale = 1.f, float *gate_t = nullptr) {
    const int lane = threadIdx.x & 31;
    float wsel = 0.f;                            // lane a keeps the weight of rank a
    if (NJ == 8) {
        // Up to 256 experts: the rounds visit the experts in ONE total order -- value descending, id ascending, every value
        // that never compares greater (NaN or <= -1e30f) in a lowest class -- so each lane sorts its eight experts by that
        // order once (19 compare-exchanges in registers) and a round only looks at the lanes' heads: two warp reductions
        // and a shift in the winning lane, instead of an eight-way scan and an eight-way update per round.
        // An expert is the pair (kh, kl) = (order-preserving key of the value or 0, ~id); a larger pair is picked earlier.
        uint32_t kh[8], kl[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int e = lane + 32 * j;
            kh[j] = 0u; kl[j] = 0u;                                         // past the end: below every expert
            if (e < E) {
                const float v = s_sb[e] + 0.0f;                             // -0 -> +0
                const uint32_t bits = __float_as_uint(v);
                if (v > -1e30f) kh[j] = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
                kl[j] = ~(uint32_t)e;
            }
        }
#define SW_CE(i, j) { const bool sw_ = kh[j] > kh[i] || (kh[j] == kh[i] && kl[j] > kl[i]);                                  \
                      const uint32_t h_ = sw_ ? kh[j] : kh[i], l_ = sw_ ? kl[j] : kl[i];                                       \
                      kh[j] = sw_ ? kh[i] : kh[j]; kl[j] = sw_ ? kl[i] : kl[j]; kh[i] = h_; kl[i] = l_; }
        SW_CE(0, 1) SW_CE(2, 3) SW_CE(4, 5) SW_CE(6, 7)
        SW_CE(0, 2) SW_CE(1, 3) SW_CE(4, 6) SW_CE(5, 7)
        SW_CE(1, 2) SW_CE(5, 6)
        SW_CE(0, 4) SW_CE(1, 5) SW_CE(2, 6) SW_CE(3, 7)
        SW_CE(2, 4) SW_CE(3, 5)
        SW_CE(1, 2) SW_CE(3, 4) SW_CE(5, 6)
#undef SW_CE
        for (int a = 0; a < K; a++) {
            const uint32_t kmax = __reduce_max_sync(SW_FULL_MASK, kh[0]);
            const uint32_t best = ~__reduce_max_sync(SW_FULL_MASK, kh[0] == kmax ? kl[0] : 0u);   // largest ~id = lowest id
            if ((int)(best & 31) == lane) {
#pragma unroll
                for (int j = 0; j < 7; j++) { kh[j] = kh[j + 1]; kl[j] = kl[j + 1]; }
                kh[7] = 0u; kl[7] = 0u;
            }
            if (lane == a) wsel = s_sc[best];
            if (lane == 0) sel_t[a] = (int)best;
        }
    } else {
    float v[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int e = lane + 32 * j;
        v[j] = e < E ? s_sb[e] + 0.0f : __int_as_float(0x7fc00000);     // -0 -> +0; past the end: NaN, never greater
    }
    uint32_t used = 0;                           // bit j: this lane's expert lane+32j is taken
    for (int a = 0; a < K; a++) {
        float bv = -1e30f; int bj = -1;
#pragma unroll
        for (int j = 0; j < NJ; j++) if (v[j] > bv) { bv = v[j]; bj = j; }
        const uint32_t bits = __float_as_uint(bv);
        const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
        const uint32_t kmax = __reduce_max_sync(SW_FULL_MASK, key);
        const uint32_t cand = (bj >= 0 && key == kmax) ? (uint32_t)(lane + 32 * bj) : 0xffffffffu;
        uint32_t best = __reduce_min_sync(SW_FULL_MASK, cand);
        if (best == 0xffffffffu) {               // nothing compared greater: lowest id not taken yet
            uint32_t c = 0xffffffffu;
#pragma unroll
            for (int j = NJ - 1; j >= 0; j--) if (lane + 32 * j < E && !(used & (1u << j))) c = (uint32_t)(lane + 32 * j);
            best = __reduce_min_sync(SW_FULL_MASK, c);
            if (best == 0xffffffffu) best = 0;
        }
        if ((int)(best & 31) == lane) {
            used |= 1u << (best >> 5);
#pragma unroll
            for (int j = 0; j < NJ; j++) if (j == (int)(best >> 5)) v[j] = __int_as_float(0x7fc00000);
        }
        if (lane == a) wsel = s_sc[best];
        if (lane == 0) sel_t[a] = (int)best;
    }
    }
    if (pool) {
        float sm = 0.f;
        for (int a = 0; a < K; a++) sm += __shfl_sync(SW_FULL_MASK, wsel, a);
        const float ws = s_sc[E];
        sm += ws;
        const float f = pool_scale / sm;
        wsel *= f;
        if (lane == 0 && gate_t) *gate_t = ws * f;
    } else if (norm_topk) {                      // float sum in rank order, then divide
        float sm = 0.f;
        for (int a = 0; a < K; a++) sm += __shfl_sync(SW_FULL_MASK, wsel, a);
        wsel = wsel / sm;
    }
    if (lane < K) w_t[lane] = wsel;
}

// One CTA of 256 threads per token.  Phase 1 (all threads, one expert each per
// pass): logits from the fp64 slice partials (or as given), gate activation,
// score and score+bias into shared memory.  Phase 2 (warp 0): the K selection
// rounds over shared memory and the combine weights.
__global__ void __launch_bounds__(256)
k_route_topk(float *__restrict__ scores, const double *__restrict__ part, int KS, const float *__restrict__ lbias,
             const float *__restrict__ corr_bias, int use_bias,
             int route_act, int norm_topk, int T, int E, int K,
             int *__restrict__ sel, float *__restrict__ w, SwRouting dr, unsigned *ticket,
             int ns, float pool_scale, float *__restrict__ row_gate) {
    extern __shared__ int sw_dyn_i[];
    __shared__ float s_sc[SW_MAX_EXPERTS], s_sb[SW_MAX_EXPERTS];
    __shared__ int s_last;
    __shared__ float s_redf[8];
    __shared__ double s_redd[8];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // ns = 1: the router has one more row, the shared expert's logit (sigmoid gate only); it takes no part in the selection
    const int ET = E + ns;
    float *r = scores + (size_t)t * ET;
    const bool ub = use_bias && corr_bias != nullptr;

    // logits
    for (int e = tid; e < ET; e += 256) {
        float v;
        if (part) {
            // slice partials are loaded 32 or eight at a time (independent loads) and added in slice order
            double a = 0.0;
            const double *pp = part + (size_t)t * ET + e;
            const size_t stride = (size_t)T * ET;
            int ks = 0;
            for (; ks + 32 <= KS; ks += 32) {
                double p[32];
#pragma unroll
                for (int i = 0; i < 32; i++) p[i] = pp[(size_t)(ks + i) * stride];
#pragma unroll
                for (int i = 0; i < 32; i++) a += p[i];
            }
            for (; ks + 8 <= KS; ks += 8) {
                double p[8];
#pragma unroll
                for (int i = 0; i < 8; i++) p[i] = pp[(size_t)(ks + i) * stride];
#pragma unroll
                for (int i = 0; i < 8; i++) a += p[i];
            }
            for (; ks < KS; ks++) a += pp[(size_t)ks * stride];
            v = (float)a;
            if (lbias && e < E) v += lbias[e];
        } else v = r[e];
        s_sc[e] = v;
    }
    __syncthreads();

    if (route_act == 1) {                        // softmax_row: float max, exp, double sum in index order per thread, 1/sum
        float m = -INFINITY;
        for (int e = tid; e < E; e += 256) { float v = s_sc[e]; if (v > m) m = v; }
#pragma unroll
        for (int off = 16; off; off >>= 1) { float o = __shfl_xor_sync(SW_FULL_MASK, m, off); if (o > m) m = o; }
        if (lane == 0) s_redf[warp] = m;
        __syncthreads();
        m = s_redf[0];
#pragma unroll
        for (int i = 1; i < 8; i++) if (s_redf[i] > m) m = s_redf[i];
        const float r0 = s_sc[0];
        if (r0 != r0) m = r0;                    // the reference's max starts from x[0]: a NaN there sticks
        double sum = 0.0;
        for (int e = tid; e < E; e += 256) { float v = sw_expf_cr(s_sc[e] - m); s_sb[e] = v; sum += (double)v; }
#pragma unroll
        for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(SW_FULL_MASK, sum, off);
        if (lane == 0) s_redd[warp] = sum;
        __syncthreads();
        sum = 0.0;
#pragma unroll
        for (int i = 0; i < 8; i++) sum += s_redd[i];
        const float inv = (float)(1.0 / sum);
        for (int e = tid; e < E; e += 256) s_sc[e] = s_sb[e] * inv;
    } else if (route_act == 0) {                 // sigmoid
        for (int e = tid; e < ET; e += 256) s_sc[e] = 1.f / (1.f + sw_expf_cr(-s_sc[e]));
    } else {                                     // softplus
        for (int e = tid; e < E; e += 256) {
            const float v = s_sc[e];
            s_sc[e] = v > 20.f ? v : (float)log1p((double)sw_expf_cr(v));
        }
    }
    __syncthreads();
    for (int e = tid; e < ET; e += 256) {
        const float sc = s_sc[e];
        r[e] = sc;                               // keep the scores for inspection
        if (e < E) s_sb[e] = sc + (ub ? corr_bias[e] : 0.f);
    }
    __syncthreads();
    if (warp == 0) {
        const int nj = (E + 31) >> 5;
        const bool pool = ns > 0;
        float *gt = row_gate ? row_gate + t : nullptr;
        if (nj <= 8) sw_topk_warp<8>(s_sb, s_sc, E, K, norm_topk, sel + (size_t)t * K, w + (size_t)t * K, pool, pool_scale, gt);
        else if (nj <= 16) sw_topk_warp<16>(s_sb, s_sc, E, K, norm_topk, sel + (size_t)t * K, w + (size_t)t * K, pool, pool_scale, gt);
        else sw_topk_warp<32>(s_sb, s_sc, E, K, norm_topk, sel + (size_t)t * K, w + (size_t)t * K, pool, pool_scale, gt);
    }
    if (!ticket) return;

    // The CTA that finishes last groups all T*K pairs by expert (saves a launch on the critical path).
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *ticket = 0;                   // every other CTA has drawn its ticket: ready for the next call
    sw_dispatch_block<256>(sw_dyn_i, dr.sel, T * K, K, E, T, dr.G, dr.gexp, dr.gbeg, dr.gcnt, dr.grow, dr.rowof, dr.status);
}

// dr/ticket non-null: the last CTA also runs the dispatch (ticket must be zero before the first call; it is
// left at zero again).
int sw_launch_route_topk(const SwLaunchCfg &c, float *scores, const double *part, int KS, const float *lbias,
                         const float *corr_bias, int use_bias,
                         int route_act, int norm_topk, int T, int E, int K, int *sel, float *w,
                         const SwRouting *dr, unsigned *ticket, int ns, float pool_scale, float *row_gate) {
    if (T <= 0) return 0;
    if (E + ns > SW_MAX_EXPERTS || K > SW_MAX_TOPK || K > E || K <= 0 || ns < 0 || ns > 1 || (ns && route_act != 0)) return -1;
    static SwPerDevice attr_done;
    if (attr_done.get(c.dev, [] {
            if (cudaFuncSetAttribute(k_route_topk, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    SwRouting none{};
    const bool fuse = dr && ticket;
    size_t smem = fuse ? (size_t)(256 / 32 + 2) * E * sizeof(int) : 0;
    k_route_topk<<<T, 256, smem, c.stream>>>(scores, part, KS, lbias, corr_bias, use_bias, route_act, norm_topk, T, E, K, sel, w,
                                             fuse ? *dr : none, fuse ? ticket : nullptr, ns, pool_scale, row_gate);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

#define SW_DISPATCH_THREADS 1024

__global__ void __launch_bounds__(SW_DISPATCH_THREADS)
k_dispatch(const int *__restrict__ sel, int npairs, int K, int E, int T,
           int *__restrict__ Gout, int *__restrict__ gexp, int *__restrict__ gbeg, int *__restrict__ gcnt,
           int *__restrict__ grow, int *__restrict__ rowof, int *__restrict__ status) {
    extern __shared__ int sm[];
    sw_dispatch_block<SW_DISPATCH_THREADS>(sm, sel, npairs, K, E, T, Gout, gexp, gbeg, gcnt, grow, rowof, status);
}

// ---------------------------------------------------------------------------
// The same grouping for many pairs (prefill), by many CTAs in three launches.
// A segment is DP_SEG consecutive pairs, walked by one warp; a CTA has eight.
//   k_dpar_hist     per-segment histograms            hist[e][s]
//   k_dpar_scan     a warp per expert: exclusive scan over the segments (the first slot, inside the expert's group, of
//                   each segment's pairs) and the expert's total; the last CTA to finish (ticket) scans the totals
//                   over the experts and writes the group arrays, exactly as the one-CTA version does
//   k_dpar_scatter  per segment, in pair order, with __match_any ranks: slot = pos[e] + hist[e][s] + rank
// Pairs of one expert therefore keep ascending flat index: the reference's order (c/laguna.c:709-723), bit for bit.
// Scratch: [ticket, 31 unused][cnt E][pos E][hist E x NSP].
// ---------------------------------------------------------------------------
#define DP_SEG 256
#define DP_WARPS 8
#define DP_MIN_PAIRS 16384         // below this one CTA is as fast (and is fused into the top-k kernel below 4096)

size_t sw_dispatch_scratch_ints(size_t P, size_t E) {
    const size_t nb = (P + DP_SEG * DP_WARPS - 1) / (DP_SEG * DP_WARPS);
    return 32 + 2 * E + E * nb * DP_WARPS;
}

__global__ void __launch_bounds__(DP_WARPS * 32)
k_dpar_hist(const int *__restrict__ sel, int npairs, int E, int NSP, int *__restrict__ hist, int *__restrict__ status) {
    extern __shared__ int dp_sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *wh = dp_sm + warp * E;
    for (int e = lane; e < E; e += 32) wh[e] = 0;
    __syncwarp();
    const int s = blockIdx.x * DP_WARPS + warp;
    const int s0 = min(s * DP_SEG, npairs), s1 = min(s0 + DP_SEG, npairs);
    for (int i = s0 + lane; i < s1; i += 32) {
        const int e = __ldcg(sel + i);
        if (e == SW_NO_EXPERT) continue;
        if (e < 0 || e >= E) { atomicOr(status, SW_ST_BAD_EXPERT); continue; }
        atomicAdd(&wh[e], 1);
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) hist[(size_t)e * NSP + s] = wh[e];
}

__global__ void __launch_bounds__(256)
k_dpar_scan(int E, int NSP, int *__restrict__ hist, int *__restrict__ cnt, int *__restrict__ pos, unsigned *__restrict__ ticket,
            int *__restrict__ Gout, int *__restrict__ gexp, int *__restrict__ gbeg, int *__restrict__ gcnt) {
    __shared__ int s_last, s_wsum[8], s_gsum[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int e = blockIdx.x * 8 + warp;
    if (e < E) {
        int carry = 0;
        int *row = hist + (size_t)e * NSP;
        for (int base = 0; base < NSP; base += 32) {
            const int i = base + lane;
            const int v = i < NSP ? row[i] : 0;
            int inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) { const int a = __shfl_up_sync(SW_FULL_MASK, inc, off); if (lane >= off) inc += a; }
            if (i < NSP) row[i] = carry + inc - v;
            carry += __shfl_sync(SW_FULL_MASK, inc, 31);
        }
        if (lane == 0) cnt[e] = carry;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *ticket = 0;
    // exclusive scan over the experts of cnt (slots) and of cnt > 0 (group index): every thread owns a run of CH experts
    const int CH = (E + 255) / 256;
    const int e0 = min(E, tid * CH), e1 = min(E, e0 + CH);
    int c = 0, nz = 0;
    for (int x = e0; x < e1; x++) { const int v = __ldcg(cnt + x); c += v; nz += v > 0 ? 1 : 0; }
    int sc = c, sg = nz;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(SW_FULL_MASK, sc, off), b = __shfl_up_sync(SW_FULL_MASK, sg, off);
        if (lane >= off) { sc += a; sg += b; }
    }
    if (lane == 31) { s_wsum[warp] = sc; s_gsum[warp] = sg; }
    __syncthreads();
    int wbase = 0, gbase = 0;
    for (int wv = 0; wv < warp; wv++) { wbase += s_wsum[wv]; gbase += s_gsum[wv]; }
    int excl = wbase + sc - c, gidx = gbase + sg - nz;
    for (int x = e0; x < e1; x++) {
        const int ce = __ldcg(cnt + x);
        pos[x] = excl;
        if (ce > 0) { gexp[gidx] = x; gbeg[gidx] = excl; gcnt[gidx] = ce; gidx++; }
        excl += ce;
    }
    if (tid == 255) { Gout[0] = gidx; Gout[1] = excl; }          // groups, and pairs that selected an expert
}

__global__ void __launch_bounds__(DP_WARPS * 32)
k_dpar_scatter(const int *__restrict__ sel, int npairs, int K, int E, int T, int NSP, const int *__restrict__ hist,
               const int *__restrict__ pos, int *__restrict__ grow, int *__restrict__ rowof, int *__restrict__ status) {
    extern __shared__ int dp_sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *wh = dp_sm + warp * E;                                  // next slot of each expert for this segment
    const int s = blockIdx.x * DP_WARPS + warp;
    for (int e = lane; e < E; e += 32) wh[e] = pos[e] + hist[(size_t)e * NSP + s];
    __syncwarp();
    const int s0 = min(s * DP_SEG, npairs), s1 = min(s0 + DP_SEG, npairs);
    for (int base = s0; base < s1; base += 32) {
        const int i = base + lane;
        const int e = i < s1 ? __ldcg(sel + i) : -1;
        const bool ok = e >= 0 && e < E;
        const unsigned peers = __match_any_sync(SW_FULL_MASK, ok ? e : -1 - lane);
        const int first = ok ? wh[e] : 0;
        __syncwarp();
        if (ok) {
            const int rank = __popc(peers & ((1u << lane) - 1));
            const int slot = first + rank, row = i / K;
            if (row >= T) atomicOr(status, SW_ST_BAD_ROW);
            else { grow[slot] = row; rowof[i] = slot; }
            if (rank == 0) wh[e] = first + __popc(peers);
        }
        __syncwarp();
    }
}

int sw_launch_dispatch(const SwLaunchCfg &c, const SwRouting &r, int T, int K, int E) {
    if (T <= 0) return 0;
    if (E > SW_MAX_EXPERTS) return -1;
    const long long npairs = (long long)T * K;
    if (r.dpar && npairs >= DP_MIN_PAIRS && sw_dispatch_scratch_ints((size_t)npairs, (size_t)E) <= r.dpar_ints) {
        const int NB = (int)((npairs + DP_SEG * DP_WARPS - 1) / (DP_SEG * DP_WARPS)), NSP = NB * DP_WARPS;
        int *cnt = r.dpar + 32, *pos = cnt + E, *hist = pos + E;
        const size_t smem = (size_t)DP_WARPS * E * sizeof(int);
        k_dpar_hist<<<NB, DP_WARPS * 32, smem, c.stream>>>(r.sel, (int)npairs, E, NSP, hist, r.status);
        k_dpar_scan<<<(E + 7) / 8, 256, 0, c.stream>>>(E, NSP, hist, cnt, pos, (unsigned *)r.dpar, r.G, r.gexp, r.gbeg, r.gcnt);
        k_dpar_scatter<<<NB, DP_WARPS * 32, smem, c.stream>>>(r.sel, (int)npairs, K, E, T, NSP, hist, pos, r.grow, r.rowof, r.status);
        sw_count_launch(); sw_count_launch(); sw_count_launch();
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }
    size_t smem = (size_t)(SW_DISPATCH_THREADS / 32 + 2) * E * sizeof(int);
    static SwPerDevice attr_done;
    if (attr_done.get(c.dev, [] {
            if (cudaFuncSetAttribute(k_dispatch, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    k_dispatch<<<1, SW_DISPATCH_THREADS, smem, c.stream>>>(r.sel, T * K, K, E, T, r.G, r.gexp, r.gbeg, r.gcnt,
                                                          r.grow, r.rowof, r.status);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
