// sw_moe_route_static: routing (router logits -> gate -> top-k -> combine weights)
// for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a
// routing decision: an engine that has already handed every free byte of the GPU
// to its expert cache (a late allocation simply fails there), or a serving loop
// that cannot afford the device-wide synchronisation an allocation or a free
// implies.  For them this one entry point takes caller-owned input and output
// buffers and keeps its working memory in a fixed array that is part of the
// library image: every GPU that loads the library reserves SW_STATIC_BYTES
// (about 2.1 MB) until the process exits.
//
// It is ONE kernel: every CTA writes fp64 partial router logits for its slice of
// the contraction into the fixed array, takes a ticket from a counter in the same
// array, and the CTA that draws the last ticket sums the partials in slice order,
// applies the gate and selects the top-k.  The arithmetic and the order of the
// partial sums are those of sw_moe_route, so both give the same ids; the combine
// weights agree to the last place or one unit of it (the softmax denominator is
// reduced over 128 threads here and over 256 there).
//
// Limits (rejected with an error text, nothing is launched): T <= 8 rows,
// n_experts <= 512, D <= 8192 and D % 32 == 0.
//
// The array is shared by every call on that GPU and keeps whatever the last call
// left in it.  The ticket counter is cleared on the caller's stream before each
// launch; the partial sums are fully rewritten by each call.  Two calls that
// overlap on the GPU (different streams, no ordering between them) race on the
// array and on the counter: order them.
//
// The first call on a device looks up the device address of the array
// (cudaGetSymbolAddress) and queries the SM count; make that first call outside
// any stream capture.  Make it at start-up too: CUDA loads a module lazily, so the
// 2.1 MB are reserved when this first call touches the module, not when the
// library is loaded -- a host that gives all device memory away before its first
// call finds no room left for the array and gets -1.
#include "sw_common.cuh"
#pragma GCC visibility push(default)
#include "../../include/sabrewing_b200.h"
#pragma GCC visibility pop
#include <stdio.h>

#define SW_STATIC_MAX_T 8
#define SW_STATIC_MAX_E 512
#define SW_STATIC_MAX_D 8192
#define SW_STATIC_MAX_SLICES (SW_STATIC_MAX_D / 128)      // sw_router_slices never cuts finer than 128 columns
#define SW_STATIC_PART_BYTES ((size_t)SW_STATIC_MAX_SLICES * SW_STATIC_MAX_T * SW_STATIC_MAX_E * 8)
#define SW_STATIC_BYTES (SW_STATIC_PART_BYTES + 256)

// [fp64 partial logits: slices x T x E][ticket counter]
static __device__ __align__(256) unsigned char sw_static_scratch[SW_STATIC_BYTES];

int sw_noalloc_fail(const char *msg);            // sets the library's last-error text (sw_api.cu)

__device__ __forceinline__ void sna_load8(const float *p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void sna_load8(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4 *>(p);
    uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(u[i] << 16); v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}
__device__ __forceinline__ void sna_dmma(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c[0]), "+d"(c[1]) : "d"(a), "d"(b));
}
__device__ __forceinline__ float sna_expf(float v) { return (float)exp((double)v); }

template <typename WT>
__global__ void __launch_bounds__(128)
k_route_static(const float *__restrict__ x, const WT *__restrict__ W, const float *__restrict__ lbias,
               const float *__restrict__ corr_bias, int use_bias, int route_act, int norm_topk,
               int T, int D, int E, int K, int KS, int slice,
               double *part, unsigned *ticket, int *__restrict__ sel, float *__restrict__ w) {
    __shared__ float s_sc[SW_STATIC_MAX_E], s_sb[SW_STATIC_MAX_E];
    __shared__ float s_redf[4];
    __shared__ double s_redd[4];
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, c = lane & 3;

    // ---- partial logits: warp item = (tile of 8 experts, slice); all T <= 8 rows are one n-tile ----
    const int etiles = (E + 7) >> 3, items = etiles * KS;
    for (int item = blockIdx.x * 4 + warp; item < items; item += gridDim.x * 4) {
        const int ks = item % KS, et = item / KS;
        const int k0 = ks * slice, k1 = min(D, k0 + slice);
        const WT *wr = W + (size_t)min(et * 8 + r, E - 1) * D + c * 8;
        const float *xr = x + (size_t)min(r, T - 1) * D + c * 8;
        double acc[2] = {0.0, 0.0};
        for (int k = k0; k < k1; k += 32) {
            float wv[8], xv[8];
            sna_load8(wr + k, wv); sna_load8(xr + k, xv);
#pragma unroll
            for (int j = 0; j < 8; j++) sna_dmma(acc, (double)wv[j], (double)xv[j]);
        }
        const int eo = et * 8 + r;
        if (eo < E) {
#pragma unroll
            for (int j = 0; j < 2; j++) { const int t = 2 * c + j; if (t < T) part[((size_t)ks * T + t) * E + eo] = acc[j]; }
        }
    }
    // ---- ticket: the CTA that arrives last sees every partial sum ----
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    const bool ub = use_bias && corr_bias != nullptr;
    for (int t = 0; t < T; t++) {
        for (int e = tid; e < E; e += 128) {
            double a = 0.0;
            for (int ks = 0; ks < KS; ks++) a += __ldcg(part + ((size_t)ks * T + t) * E + e);
            float v = (float)a;
            if (lbias) v += lbias[e];
            s_sc[e] = v;
        }
        __syncthreads();
        if (route_act == 1) {
            float m = -INFINITY;
            for (int e = tid; e < E; e += 128) { float v = s_sc[e]; if (v > m) m = v; }
#pragma unroll
            for (int off = 16; off; off >>= 1) { float o = __shfl_xor_sync(SW_FULL_MASK, m, off); if (o > m) m = o; }
            if (lane == 0) s_redf[warp] = m;
            __syncthreads();
            m = s_redf[0];
#pragma unroll
            for (int i = 1; i < 4; i++) if (s_redf[i] > m) m = s_redf[i];
            const float r0 = s_sc[0];
            if (r0 != r0) m = r0;
            double sum = 0.0;
            for (int e = tid; e < E; e += 128) { float v = sna_expf(s_sc[e] - m); s_sb[e] = v; sum += (double)v; }
#pragma unroll
            for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(SW_FULL_MASK, sum, off);
            if (lane == 0) s_redd[warp] = sum;
            __syncthreads();
            sum = 0.0;
#pragma unroll
            for (int i = 0; i < 4; i++) sum += s_redd[i];
            const float inv = (float)(1.0 / sum);
            for (int e = tid; e < E; e += 128) s_sc[e] = s_sb[e] * inv;
        } else if (route_act == 0) {
            for (int e = tid; e < E; e += 128) s_sc[e] = 1.f / (1.f + sna_expf(-s_sc[e]));
        } else {
            for (int e = tid; e < E; e += 128) { const float v = s_sc[e]; s_sc[e] = v > 20.f ? v : (float)log1p((double)sna_expf(v)); }
        }
        __syncthreads();
        for (int e = tid; e < E; e += 128) s_sb[e] = s_sc[e] + (ub ? corr_bias[e] : 0.f);
        __syncthreads();
        if (warp == 0) {
            uint32_t used = 0; float wsel = 0.f;
            for (int a = 0; a < K; a++) {
                float bv = -1e30f; int best = -1, j = 0;
                for (int e = lane; e < E; e += 32, j++) {
                    if (used & (1u << j)) continue;
                    const float s = s_sb[e];
                    if (s > bv) { bv = s; best = e; }
                }
#pragma unroll
                for (int off = 16; off; off >>= 1) {
                    float ov = __shfl_xor_sync(SW_FULL_MASK, bv, off);
                    int oi = __shfl_xor_sync(SW_FULL_MASK, best, off);
                    if (oi >= 0 && (best < 0 || ov > bv || (ov == bv && oi < best))) { bv = ov; best = oi; }
                }
                if (best < 0) {
                    int cand = 0x7fffffff; j = 0;
                    for (int e = lane; e < E; e += 32, j++) if (!(used & (1u << j))) { cand = e; break; }
#pragma unroll
                    for (int off = 16; off; off >>= 1) { int o = __shfl_xor_sync(SW_FULL_MASK, cand, off); if (o < cand) cand = o; }
                    best = cand == 0x7fffffff ? 0 : cand;
                }
                if ((best & 31) == lane) used |= 1u << (best >> 5);
                if (lane == a) wsel = s_sc[best];
                if (lane == 0) sel[(size_t)t * K + a] = best;
            }
            if (norm_topk) {
                float sm = 0.f;
                for (int a = 0; a < K; a++) sm += __shfl_sync(SW_FULL_MASK, wsel, a);
                wsel = wsel / sm;
            }
            if (lane < K) w[(size_t)t * K + lane] = wsel;
        }
        __syncthreads();
    }
}

// per device: address of the fixed array and SM count, looked up on the first call there
static struct { void *ptr; int sms; } g_static_dev[64];

extern "C" int sw_moe_route_static(const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T,
                                   int *sel, float *w, void *stream) {
    if (!d || !L || !x || !sel || !w) return sw_noalloc_fail("route_static: null argument");
    if (T < 0 || T > SW_STATIC_MAX_T) return sw_noalloc_fail("route_static: T outside [0,8] (the fixed scratch array holds 8 rows)");
    if (d->n_experts <= 0 || d->n_experts > SW_STATIC_MAX_E) return sw_noalloc_fail("route_static: n_experts outside (0,512]");
    if (L->D <= 0 || L->D > SW_STATIC_MAX_D || L->D % 32) return sw_noalloc_fail("route_static: D must be a multiple of 32 and <= 8192");
    if (d->topk <= 0 || d->topk > SW_MAX_TOPK || d->topk > d->n_experts) return sw_noalloc_fail("route_static: bad topk");
    if (d->route_act < 0 || d->route_act > 2 || !L->router_w) return sw_noalloc_fail("route_static: bad route_act or missing router weights");
    if (L->router_dtype != SW_DTYPE_F32 && L->router_dtype != SW_DTYPE_BF16) return sw_noalloc_fail("route_static: unknown router_dtype");
    if (d->shared_mode == SW_SHARED_GATED) return sw_noalloc_fail("route_static: the shared-pool policy (SW_SHARED_GATED) is not served here");
    // x and the router rows are read with 128-bit loads
    if (((uintptr_t)x | (uintptr_t)L->router_w) & 15) return sw_noalloc_fail("route_static: x and router_w must be 16-byte aligned");
    if (((uintptr_t)sel | (uintptr_t)w | (uintptr_t)L->corr_bias | (uintptr_t)L->logit_bias) & 3) return sw_noalloc_fail("route_static: sel, w and the bias arrays must be 4-byte aligned");
    if (T == 0) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return sw_noalloc_fail("route_static: no current device"); }
    {
        // first call on this device: look the array's device address up (under the set-up mutex, so that two
        // threads making their first call at once both see a complete entry)
        std::lock_guard<std::mutex> g(sw_setup_mutex());
        if (!g_static_dev[dev].ptr) {
            void *p = nullptr; int sms = 0;
            if (cudaGetSymbolAddress(&p, sw_static_scratch) != cudaSuccess || !p) { cudaGetLastError(); return sw_noalloc_fail("route_static: cudaGetSymbolAddress failed"); }
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) { cudaGetLastError(); return sw_noalloc_fail("route_static: cannot query the device"); }
            g_static_dev[dev].sms = sms; g_static_dev[dev].ptr = p;
        }
    }
    const int E = d->n_experts;
    const int KS = sw_router_slices(g_static_dev[dev].sms, T, L->D, E);      // same slicing as sw_moe_route
    if (KS > SW_STATIC_MAX_SLICES) return sw_noalloc_fail("route_static: slice count exceeds the fixed scratch array");
    const int slice = ((L->D + KS - 1) / KS + 31) & ~31;
    double *part = (double *)g_static_dev[dev].ptr;
    unsigned *ticket = (unsigned *)((unsigned char *)g_static_dev[dev].ptr + SW_STATIC_PART_BYTES);
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(ticket, 0, sizeof(unsigned), st) != cudaSuccess) { cudaGetLastError(); return sw_noalloc_fail("route_static: clearing the ticket counter failed"); }
    const int items = ((E + 7) / 8) * KS;
    int grid = (items + 3) / 4;
    if (grid > g_static_dev[dev].sms * 8) grid = g_static_dev[dev].sms * 8;
    if (L->router_dtype == SW_DTYPE_BF16)
        k_route_static<__nv_bfloat16><<<grid, 128, 0, st>>>(x, (const __nv_bfloat16 *)L->router_w, L->logit_bias, L->corr_bias, d->use_corr_bias,
                                                            d->route_act, d->norm_topk, T, L->D, E, d->topk, KS, slice, part, ticket, sel, w);
    else
        k_route_static<float><<<grid, 128, 0, st>>>(x, (const float *)L->router_w, L->logit_bias, L->corr_bias, d->use_corr_bias,
                                                    d->route_act, d->norm_topk, T, L->D, E, d->topk, KS, slice, part, ticket, sel, w);
    sw_count_launch();
    if (cudaGetLastError() != cudaSuccess) return sw_noalloc_fail("route_static: kernel launch failed");
    return 0;
}
