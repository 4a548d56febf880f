// Expert products of the MoE block on CUDA cores with f32 activations:
// grouped int4 GEMV (gate/up with the SiLU*up epilogue, and down), the bf16
// shared expert, the int8 resident GEMV, and the rank-order combine.
//
// Reference behaviour restated here:
//   int4 dot        c/moe_quant.h:45-125 (value = nibble-8, low nibble = even column,
//                   acc * scale[o]); grouped form c/backend_cuda_laguna.cu:420-443
//   SiLU*up         c/laguna.c:747-750, siluf c/moe_math.h:53
//   bf16 residents  matmul_bf16_k round_x=0, c/moe_matmul.h:92-111
//   combine         c/laguna.c:761-771 (rank order), c/moe_block.h:37-51
#include "sw_common.cuh"

// ---------------------------------------------------------------------------
// Grouped int4 GEMV.  Work item = (group g, block of output rows).  The CTA
// stages up to NC activation rows of the group in shared memory (re-laid so that
// lane l's q-th float4 of its 32-column unit sits at float4 index q*UP+u:
// conflict-free 128-bit reads), then every warp streams RW weight rows at a time
// with 128-bit loads, dequantises in registers and accumulates NC rows at once.
// Each (row, token) dot is reduced in the same order whatever the group size, so
// grouping never changes a result bit (the reference's grouped-vs-per-token bar,
// c/laguna.c:1620-1657).
// ---------------------------------------------------------------------------
// GS: scales are per group of `gs` columns (gs % 32 == 0), laid out [row, ceil(KD/gs)] like the reference's
// group-scaled int4 (c/quant.h:167-202): each 32-column unit's partial dot is multiplied by its group's
// scale before it is accumulated, and there is no final per-row multiply.
template <bool GATEUP, int NC, bool GS>
__global__ void __launch_bounds__(256)
k_q4_group(const uint8_t *__restrict__ Wq, const float *__restrict__ Ws,
           const float *__restrict__ X, float *__restrict__ Y,
           const int *__restrict__ gexp, const int *__restrict__ gbeg, const int *__restrict__ gcnt,
           const int *__restrict__ Gp, const int *__restrict__ grow,
           int KD, int OUT, int rows_per_item, int expert_lo, int expert_cnt, int gs) {
    extern __shared__ float4 xs4[];              // [NC][8*UP] float4
    const int ng = GS ? (KD + gs - 1) / gs : 1;  // scales per weight row
    const int U = KD >> 5;                       // 32-column units per row
    const int UP = U + 1;                        // padded stride between the 8 float4 planes
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = *Gp;
    const int ipg = (OUT + rows_per_item - 1) / rows_per_item;
    const int items = G * ipg;
    const int nrows_w = GATEUP ? 2 * OUT : OUT;  // weight rows per expert
    const size_t rowbytes = (size_t)(KD >> 1);

    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int g = item / ipg, rb = item - g * ipg;
        const int e = gexp[g] - expert_lo;
        if (e < 0 || e >= expert_cnt) continue;
        const int n = gcnt[g], beg = gbeg[g];
        const uint8_t *wq = Wq + (size_t)e * nrows_w * rowbytes;
        const float *ws = Ws + (size_t)e * nrows_w * ng;
        const int r_lo = rb * rows_per_item, r_hi = min(r_lo + rows_per_item, OUT);

        for (int c0 = 0; c0 < n; c0 += NC) {
            const int nc = min(NC, n - c0);
            __syncthreads();
            for (int c = 0; c < NC; c++) {
                float4 *dst = xs4 + (size_t)c * 8 * UP;
                if (c < nc) {
                    const int src_row = GATEUP ? grow[beg + c0 + c] : (beg + c0 + c);
                    const float4 *src = reinterpret_cast<const float4 *>(X + (size_t)src_row * KD);
                    for (int i = tid; i < (KD >> 2); i += 256) dst[(i & 7) * UP + (i >> 3)] = src[i];
                } else {
                    for (int i = tid; i < (KD >> 2); i += 256) dst[(i & 7) * UP + (i >> 3)] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            __syncthreads();

            // each warp pass: gate/up = 2 output columns (4 weight rows), down = 4 rows
            constexpr int RW = 4;
            constexpr int OW = GATEUP ? 2 : 4;   // outputs per warp pass
            for (int o0 = r_lo + warp * OW; o0 < r_hi; o0 += 8 * OW) {
                const uint8_t *rp[RW]; bool rv[RW]; const float *rs[RW];
#pragma unroll
                for (int r = 0; r < RW; r++) {
                    int row, oi;
                    if (GATEUP) { oi = o0 + (r & 1); row = (r < 2 ? 0 : OUT) + oi; }
                    else        { oi = o0 + r;       row = oi; }
                    rv[r] = oi < r_hi;
                    rp[r] = wq + (size_t)(rv[r] ? row : 0) * rowbytes;
                    rs[r] = ws + (size_t)(rv[r] ? row : 0) * ng;
                }
                float acc[RW][NC];
#pragma unroll
                for (int r = 0; r < RW; r++)
#pragma unroll
                    for (int c = 0; c < NC; c++) acc[r][c] = 0.f;

                for (int u = lane; u < U; u += 32) {
                    float sgrp[RW], keep[RW][NC];
                    if (GS) {
                        const int g = (u * 32) / gs;
#pragma unroll
                        for (int r = 0; r < RW; r++) {
                            sgrp[r] = rs[r][g];
#pragma unroll
                            for (int c = 0; c < NC; c++) { keep[r][c] = acc[r][c]; acc[r][c] = 0.f; }
                        }
                    }
                    uint4 wv[RW];
#pragma unroll
                    for (int r = 0; r < RW; r++)
                        wv[r] = rv[r] ? __ldg(reinterpret_cast<const uint4 *>(rp[r]) + u) : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        float4 xv[NC];
#pragma unroll
                        for (int c = 0; c < NC; c++) xv[c] = xs4[(size_t)c * 8 * UP + q * UP + u];
#pragma unroll
                        for (int r = 0; r < RW; r++) {
                            uint32_t word = (q >> 1) == 0 ? wv[r].x : (q >> 1) == 1 ? wv[r].y : (q >> 1) == 2 ? wv[r].z : wv[r].w;
                            uint32_t h = (q & 1) ? (word >> 16) : word;
                            // nibble -> float without an int-to-float conversion: 2^23+n as bits, minus 2^23+8
                            float w0 = __uint_as_float((h & 0xFu) | 0x4B000000u) - 8388616.f;
                            float w1 = __uint_as_float(((h >> 4) & 0xFu) | 0x4B000000u) - 8388616.f;
                            float w2 = __uint_as_float(((h >> 8) & 0xFu) | 0x4B000000u) - 8388616.f;
                            float w3 = __uint_as_float(((h >> 12) & 0xFu) | 0x4B000000u) - 8388616.f;
#pragma unroll
                            for (int c = 0; c < NC; c++) {
                                acc[r][c] = fmaf(xv[c].x, w0, acc[r][c]);
                                acc[r][c] = fmaf(xv[c].y, w1, acc[r][c]);
                                acc[r][c] = fmaf(xv[c].z, w2, acc[r][c]);
                                acc[r][c] = fmaf(xv[c].w, w3, acc[r][c]);
                            }
                        }
                    }
                    if (GS) {
#pragma unroll
                        for (int r = 0; r < RW; r++)
#pragma unroll
                            for (int c = 0; c < NC; c++) acc[r][c] = fmaf(acc[r][c], sgrp[r], keep[r][c]);
                    }
                }
#pragma unroll
                for (int r = 0; r < RW; r++)
#pragma unroll
                    for (int c = 0; c < NC; c++) {
                        float a = acc[r][c];
#pragma unroll
                        for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(SW_FULL_MASK, a, off);
                        acc[r][c] = a;
                    }
                if (lane == 0) {
                    if (GATEUP) {
#pragma unroll
                        for (int p = 0; p < 2; p++) {
                            const int oi = o0 + p;
                            if (oi < r_hi) {
                                const float sg = GS ? 1.f : ws[oi], su = GS ? 1.f : ws[OUT + oi];
#pragma unroll
                                for (int c = 0; c < NC; c++) if (c < nc) {
                                    float gv = acc[p][c] * sg, uv = acc[2 + p][c] * su;
                                    Y[(size_t)(beg + c0 + c) * OUT + oi] = (gv / (1.f + expf(-gv))) * uv;
                                }
                            }
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < RW; r++) {
                            const int oi = o0 + r;
                            if (oi < r_hi) {
                                const float s = GS ? 1.f : ws[oi];
#pragma unroll
                                for (int c = 0; c < NC; c++) if (c < nc)
                                    Y[(size_t)(beg + c0 + c) * OUT + oi] = acc[r][c] * s;
                            }
                        }
                    }
                }
            }
        }
    }
}

template <bool GATEUP>
static int sw_launch_q4(const SwLaunchCfg &c, const SwQ4Args &a) {
    if (a.max_groups <= 0 || a.max_rows <= 0) return 0;
    if (a.KD % 32 || a.KD <= 0 || a.OUT <= 0) return -1;
    constexpr int NC = 4;
    const int U = a.KD / 32;
    size_t smem = (size_t)NC * 8 * (U + 1) * sizeof(float4);
    if (smem > 220 * 1024) return -1;
    if (a.gs < 0 || (a.gs > 0 && a.gs % 32)) return -1;
    auto kern = a.gs > 0 ? k_q4_group<GATEUP, NC, true> : k_q4_group<GATEUP, NC, false>;
    // the opt-in covers the largest size this kernel can be given here (220 KB), set once per device
    static SwPerDevice attr[2];
    if (attr[a.gs > 0].get(c.dev, [&] {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    // rows per work item: enough items to fill the machine a few times over, but
    // never below one pass of the 8 warps.
    const int pass = GATEUP ? 16 : 32;
    int target_items = c.num_sms * 6;
    int rpi = pass;
    while (rpi * 2 <= a.OUT && (long long)a.max_groups * ((a.OUT + rpi * 2 - 1) / (rpi * 2)) >= target_items) rpi *= 2;
    long long items = (long long)a.max_groups * ((a.OUT + rpi - 1) / rpi);
    int bps = smem <= 48 * 1024 ? 4 : smem <= 72 * 1024 ? 3 : smem <= 110 * 1024 ? 2 : 1;
    long long grid = (long long)c.num_sms * bps;
    if (grid > items) grid = items;
    if (grid < 1) grid = 1;
    kern<<<(unsigned)grid, 256, smem, c.stream>>>(a.q, a.s, a.X, a.Y, a.gexp, a.gbeg, a.gcnt, a.G, a.grow,
                                                  a.KD, a.OUT, rpi, a.expert_lo, a.expert_cnt, a.gs);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int sw_launch_q4_gateup(const SwLaunchCfg &c, const SwQ4Args &a) { return sw_launch_q4<true>(c, a); }
int sw_launch_q4_down(const SwLaunchCfg &c, const SwQ4Args &a) { return sw_launch_q4<false>(c, a); }

// ---------------------------------------------------------------------------
// bf16 resident GEMV over T rows: one warp per output row, TT token rows per
// pass; weights expanded exactly, activations f32.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void sw_bf16x8(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
    uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(u[i] << 16); v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}

template <bool GATEUP, int TT>
__global__ void __launch_bounds__(256)
k_bf16_rows(const float *__restrict__ x, const __nv_bfloat16 *__restrict__ W0, const __nv_bfloat16 *__restrict__ W1,
            float *__restrict__ y, int T, int I, int O) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * TT;
    if (o >= O) return;
    float a0[TT], a1[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) { a0[t] = 0.f; a1[t] = 0.f; }
    const __nv_bfloat16 *w0 = W0 + (size_t)o * I, *w1 = GATEUP ? W1 + (size_t)o * I : nullptr;
    for (int k = lane * 8; k < I; k += 256) {
        float wv0[8], wv1[8];
        sw_bf16x8(w0 + k, wv0);
        if (GATEUP) sw_bf16x8(w1 + k, wv1);
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (t0 + t < T) {
                const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)(t0 + t) * I + k);
                float4 xa = xp[0], xb = xp[1];
                float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    a0[t] = fmaf(xv[i], wv0[i], a0[t]);
                    if (GATEUP) a1[t] = fmaf(xv[i], wv1[i], a1[t]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        float g = a0[t], u = a1[t];
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            g += __shfl_xor_sync(SW_FULL_MASK, g, off);
            if (GATEUP) u += __shfl_xor_sync(SW_FULL_MASK, u, off);
        }
        if (lane == 0 && t0 + t < T)
            y[(size_t)(t0 + t) * O + o] = GATEUP ? (g / (1.f + expf(-g))) * u : g;
    }
}

int sw_launch_bf16_gateup(const SwLaunchCfg &c, const float *x, const void *Wg, const void *Wu,
                          float *sglu, int T, int D, int SI) {
    if (T <= 0 || SI <= 0) return 0;
    if (D % 8) return -1;
    constexpr int TT = 4;
    dim3 grid((SI + 7) / 8, (T + TT - 1) / TT);
    k_bf16_rows<true, TT><<<grid, 256, 0, c.stream>>>(x, (const __nv_bfloat16 *)Wg, (const __nv_bfloat16 *)Wu, sglu, T, D, SI);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int sw_launch_bf16_rows(const SwLaunchCfg &c, const float *x, const void *W, float *y, int T, int I, int O) {
    if (T <= 0 || O <= 0) return 0;
    if (I % 8) return -1;
    constexpr int TT = 4;
    dim3 grid((O + 7) / 8, (T + TT - 1) / TT);
    k_bf16_rows<false, TT><<<grid, 256, 0, c.stream>>>(x, (const __nv_bfloat16 *)W, nullptr, y, T, I, O);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// int8 resident GEMV, W = [int8 O*I], scale f32 [O] (c/laguna.c:135-139 layout).
template <int TT>
__global__ void __launch_bounds__(256)
k_q8_rows(const float *__restrict__ x, const int8_t *__restrict__ W, const float *__restrict__ scale,
          float *__restrict__ y, int T, int I, int O) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * TT;
    if (o >= O) return;
    float a[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) a[t] = 0.f;
    const int8_t *w = W + (size_t)o * I;
    for (int k = lane * 4; k < I; k += 128) {
        int wv = 0;
        if (k + 4 <= I && ((reinterpret_cast<uintptr_t>(w + k) & 3) == 0)) wv = *reinterpret_cast<const int *>(w + k);
        else for (int i = 0; i < 4 && k + i < I; i++) wv |= ((int)(uint8_t)w[k + i]) << (8 * i);
#pragma unroll
        for (int t = 0; t < TT; t++) if (t0 + t < T) {
            const float *xp = x + (size_t)(t0 + t) * I + k;
#pragma unroll
            for (int i = 0; i < 4; i++) if (k + i < I) a[t] = fmaf(xp[i], (float)(int8_t)(wv >> (8 * i)), a[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        float s = a[t];
#pragma unroll
        for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(SW_FULL_MASK, s, off);
        if (lane == 0 && t0 + t < T) y[(size_t)(t0 + t) * O + o] = s * scale[o];
    }
}
int sw_launch_q8_rows(const SwLaunchCfg &c, const float *x, const int8_t *W, const float *scale,
                      float *y, int T, int I, int O) {
    if (T <= 0 || O <= 0) return 0;
    constexpr int TT = 4;
    dim3 grid((O + 7) / 8, (T + TT - 1) / TT);
    k_q8_rows<TT><<<grid, 256, 0, c.stream>>>(x, W, scale, y, T, I, O);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// Rank-order combine: acc = sum_a fma(w[t,a], slots[rowof[t,a]], acc) for a = 0..K-1
// (the reference's multiply-add, contracted by its build), then optionally
// *route_scale, + add rows, and store or accumulate.
// ---------------------------------------------------------------------------
// NB ranks of one token, starting at flat pair index `base`: indices and weights first, then all slot rows (independent,
// unconditional loads: a rank whose expert lives elsewhere reads row 0 and is not added), then the FMAs in rank order.
template <int NB>
__device__ __forceinline__ void sw_combine_round(float4 &acc, const float *__restrict__ slots, const int *__restrict__ rowof,
                                                 const int *__restrict__ sel, const float *__restrict__ w, size_t base,
                                                 int D, int i4, int expert_lo, int expert_cnt, float b2) {
    float wa[NB]; int slot[NB];
#pragma unroll
    for (int j = 0; j < NB; j++) {
        const int e = sel[base + j] - expert_lo;
        const bool ok = e >= 0 && e < expert_cnt;
        const int ro = rowof[base + j];
        const float wj = w[base + j];
        slot[j] = ok ? ro : -1; wa[j] = wj * b2;
    }
    float4 v[NB];
#pragma unroll
    for (int j = 0; j < NB; j++) v[j] = reinterpret_cast<const float4 *>(slots + (size_t)max(slot[j], 0) * D)[i4];
#pragma unroll
    for (int j = 0; j < NB; j++)
        if (slot[j] >= 0) {
            acc.x = fmaf(wa[j], v[j].x, acc.x); acc.y = fmaf(wa[j], v[j].y, acc.y);
            acc.z = fmaf(wa[j], v[j].z, acc.z); acc.w = fmaf(wa[j], v[j].w, acc.w);
        }
}

template <int KB>          // ranks whose slot rows are in flight at once: 8, or 16 at decode sizes (top-k up to 16 in one round)
__global__ void __launch_bounds__(256)
k_combine(const float *__restrict__ slots, const int *__restrict__ rowof, const int *__restrict__ sel,
          const float *__restrict__ w, const float *__restrict__ add, int add_slices, float *__restrict__ out,
          int T, int K, int D, float route_scale, int mode, int expert_lo, int expert_cnt, const float *__restrict__ row_gate,
          const float *__restrict__ row_back) {
    const int D4 = D >> 2;
    const size_t n = (size_t)T * D4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / D4), i4 = (int)(idx - (size_t)t * D4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        // The tcgen05 expert kernels worked on the token row divided by the power of two row_back[t] and left the slot rows
        // divided by its square: the weights carry it back (a power of two: every product and sum scales exactly).
        float b2 = 1.f;
        if (row_back) { const float b = row_back[t]; b2 = b * b; }
        const size_t base = (size_t)t * K;
        int a0 = 0;
        for (; a0 + KB <= K; a0 += KB) sw_combine_round<KB>(acc, slots, rowof, sel, w, base + a0, D, i4, expert_lo, expert_cnt, b2);
#define SW_CR(N) case N: sw_combine_round<N>(acc, slots, rowof, sel, w, base + a0, D, i4, expert_lo, expert_cnt, b2); break;
        switch (K - a0) {                        // the remaining ranks in one round of exactly that width
            SW_CR(1) SW_CR(2) SW_CR(3) SW_CR(4) SW_CR(5) SW_CR(6) SW_CR(7)
            default:
                if (KB > 8) switch (K - a0) { SW_CR(8) SW_CR(9) SW_CR(10) SW_CR(11) SW_CR(12) SW_CR(13) SW_CR(14) SW_CR(15) default: break; }
                break;
        }
#undef SW_CR
        if (mode & 1) { acc.x *= route_scale; acc.y *= route_scale; acc.z *= route_scale; acc.w *= route_scale; }
        if (mode & 2) {
            float4 s = reinterpret_cast<const float4 *>(add)[idx];
#pragma unroll 8
            for (int k = 1; k < add_slices; k++) {
                const float4 s2 = reinterpret_cast<const float4 *>(add)[(size_t)k * n + idx];
                s.x += s2.x; s.y += s2.y; s.z += s2.z; s.w += s2.w;
            }
            if (row_gate) { const float gt = row_gate[t]; s.x *= gt; s.y *= gt; s.z *= gt; s.w *= gt; }   // gated shared expert
            acc.x += s.x; acc.y += s.y; acc.z += s.z; acc.w += s.w;
        }
        float4 *o = reinterpret_cast<float4 *>(out) + idx;
        if (mode & 4) { float4 h = *o; acc.x = h.x + acc.x; acc.y = h.y + acc.y; acc.z = h.z + acc.z; acc.w = h.w + acc.w; }
        *o = acc;
    }
}

int sw_launch_combine(const SwLaunchCfg &c, const float *slots, const int *rowof, const int *sel,
                      const float *w, const float *add, int add_slices, float *out, int T, int K, int D,
                      float route_scale, int mode, int expert_lo, int expert_cnt, const float *row_gate, const float *row_back) {
    if (T <= 0) return 0;
    if (D % 4) return -1;
    size_t n = (size_t)T * (D / 4);
    long long grid = (long long)((n + 255) / 256);
    if (grid > (long long)c.num_sms * 16) grid = (long long)c.num_sms * 16;
    // one round for top-k up to 16 when the step is latency-bound (few rows); with many rows the registers of a wide
    // round cost more than a second round does
    if (T > 64)
        k_combine<8><<<(unsigned)grid, 256, 0, c.stream>>>(slots, rowof, sel, w, add, add_slices, out, T, K, D, route_scale, mode, expert_lo, expert_cnt, row_gate, row_back);
    else
        k_combine<16><<<(unsigned)grid, 256, 0, c.stream>>>(slots, rowof, sel, w, add, add_slices, out, T, K, D, route_scale, mode, expert_lo, expert_cnt, row_gate, row_back);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// out += routed*route_scale (+ add)
__global__ void __launch_bounds__(256)
k_finish(const float *__restrict__ routed, const float *__restrict__ add, int add_slices, float *__restrict__ out,
         size_t n4, float route_scale, int has_add, const float *__restrict__ row_gate, int D4) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n4; idx += (size_t)gridDim.x * blockDim.x) {
        float4 a = reinterpret_cast<const float4 *>(routed)[idx];
        a.x *= route_scale; a.y *= route_scale; a.z *= route_scale; a.w *= route_scale;
        if (has_add) {
            float4 s = reinterpret_cast<const float4 *>(add)[idx];
            for (int k = 1; k < add_slices; k++) {
                const float4 s2 = reinterpret_cast<const float4 *>(add)[(size_t)k * n4 + idx];
                s.x += s2.x; s.y += s2.y; s.z += s2.z; s.w += s2.w;
            }
            if (row_gate) { const float gt = row_gate[idx / D4]; s.x *= gt; s.y *= gt; s.z *= gt; s.w *= gt; }
            a.x += s.x; a.y += s.y; a.z += s.z; a.w += s.w;
        }
        float4 h = reinterpret_cast<float4 *>(out)[idx];
        h.x += a.x; h.y += a.y; h.z += a.z; h.w += a.w;
        reinterpret_cast<float4 *>(out)[idx] = h;
    }
}
int sw_launch_finish(const SwLaunchCfg &c, const float *routed, const float *add, int add_slices, float *out,
                     int T, int D, float route_scale, int has_add, const float *row_gate) {
    if (T <= 0) return 0;
    if (D % 4) return -1;
    size_t n4 = (size_t)T * (D / 4);
    long long grid = (long long)((n4 + 255) / 256);
    if (grid > (long long)c.num_sms * 16) grid = (long long)c.num_sms * 16;
    k_finish<<<(unsigned)grid, 256, 0, c.stream>>>(routed, add, add_slices, out, n4, route_scale, has_add, row_gate, D / 4);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// RMSNorm of rows, the reference's rmsnorm_row (c/moe_math.h:58-62): sum of squares in double, inv = 1 / sqrtf(
// (float)(ss / D) + eps), y = x * inv * w.  One CTA per row; the double partial sums are reduced in a fixed tree.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_rmsnorm_rows(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ y, int T, int D, float eps) {
    __shared__ double s_part[8];
    __shared__ float s_inv;
    for (int r = blockIdx.x; r < T; r += gridDim.x) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)r * D);
        double ss = 0.0;
        for (int i = threadIdx.x; i < (D >> 2); i += 256) {
            const float4 v = xr[i];
            ss += (double)v.x * v.x; ss += (double)v.y * v.y; ss += (double)v.z * v.z; ss += (double)v.w * v.w;
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(SW_FULL_MASK, ss, off);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
#pragma unroll
            for (int i = 0; i < 8; i++) t += s_part[i];
            s_inv = 1.f / sqrtf((float)(t / D) + eps);
        }
        __syncthreads();
        const float inv = s_inv;
        const float4 *wr = reinterpret_cast<const float4 *>(w);
        float4 *yr = reinterpret_cast<float4 *>(y + (size_t)r * D);
        for (int i = threadIdx.x; i < (D >> 2); i += 256) {
            const float4 v = xr[i], g = wr[i];
            yr[i] = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
    }
}
int sw_launch_rmsnorm(const SwLaunchCfg &c, const float *x, const float *w, float *y, int T, int D, float eps) {
    if (T <= 0) return 0;
    if (D % 4) return -1;
    const int grid = T < c.num_sms * 8 ? T : c.num_sms * 8;
    k_rmsnorm_rows<<<grid, 256, 0, c.stream>>>(x, w, y, T, D, eps);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// y[i] = sum over the slices, in slice order, of part[k][i]
__global__ void __launch_bounds__(256)
k_sum_slices(const float *__restrict__ part, int KS, size_t n4, float *__restrict__ y) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n4; idx += (size_t)gridDim.x * blockDim.x) {
        float4 a = reinterpret_cast<const float4 *>(part)[idx];
        for (int k = 1; k < KS; k++) {
            const float4 b = reinterpret_cast<const float4 *>(part)[(size_t)k * n4 + idx];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        reinterpret_cast<float4 *>(y)[idx] = a;
    }
}
int sw_launch_sum_slices(const SwLaunchCfg &c, const float *part, int KS, size_t n, float *y) {
    if (!n) return 0;
    if (n % 4) return -1;
    const size_t n4 = n / 4;
    long long grid = (long long)((n4 + 255) / 256);
    if (grid > (long long)c.num_sms * 8) grid = (long long)c.num_sms * 8;
    k_sum_slices<<<(unsigned)grid, 256, 0, c.stream>>>(part, KS, n4, y);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// row_gate[t] = 1 / (1 + expf(-(float)(x[t] . g))): the one-row sigmoid gate of a shared expert (the reference's
// qwen35 engine, c/qwen35.c:689-697: matmul_f32 in its exact mode, i.e. a double dot rounded to f32, then the gate).
// One warp per row, fp64 partial sums reduced in a fixed tree.
__global__ void __launch_bounds__(256)
k_row_gate(const float *__restrict__ x, const float *__restrict__ g, float *__restrict__ row_gate, int T, int D) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)t * D), *gr = reinterpret_cast<const float4 *>(g);
    double a = 0.0;
    for (int i = lane; i < (D >> 2); i += 32) {
        const float4 v = xr[i], w = gr[i];
        a = fma((double)v.x, (double)w.x, a); a = fma((double)v.y, (double)w.y, a);
        a = fma((double)v.z, (double)w.z, a); a = fma((double)v.w, (double)w.w, a);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(SW_FULL_MASK, a, off);
    if (lane == 0) { const float gv = (float)a; row_gate[t] = 1.f / (1.f + (float)exp(-(double)gv)); }
}
int sw_launch_row_gate(const SwLaunchCfg &c, const float *x, const float *g, float *row_gate, int T, int D) {
    if (T <= 0) return 0;
    if (D % 4) return -1;
    k_row_gate<<<(T + 7) / 8, 256, 0, c.stream>>>(x, g, row_gate, T, D);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
