// fp4 (e2m1 codes + one ue8m0 exponent byte per 32 input columns) products for the lag_cuda_* tier:
// the dense y = x * dequant(W)^T and the fused K-expert decode step with DeepSeek-V4's clamped SwiGLU.
// Container and value mapping: c/moe_quant.h:219-257; reference kernels c/backend_cuda_laguna.cu:284-397.
//
// These calls serve single-token decode from host buffers, so the weight stream is short (K experts) and the
// kernels run on CUDA cores: a warp owns RW output rows, a lane one 16-byte piece (32 columns = exactly one
// scale block) of each row per step; the token row is read through L1 once for all RW rows.
// A code is turned into its value without a table: the four bits s e1 e0 m, placed at fp16 bits 15, 11..10
// and 9, are the fp16 number value * 2^-14 (e = 0 gives the subnormal m * 2^-15), so value = fp16 * 16384.
#include "sw_common.cuh"
#include <cuda_fp16.h>

// rows per warp (gate/up: row pairs, i.e. twice as many weight rows; fewer of them keep the register count,
// and with it the number of resident warps, where the plain rows are)
#define SW_FP4_RW(GLU) ((GLU) ? 2 : 4)
#define SW_FP4_WARPS 8

// 2^(e-127); 0xFF (the format's NaN) -> 0, 0 -> the denormal 2^-127 (c/moe_quant.h:250-256)
__device__ __forceinline__ float sw_ue8m0(unsigned e) {
    if (e == 0xFFu) return 0.f;
    if (e == 0u) return 5.8774717541114375e-39f;
    return __int_as_float((int)(e << 23));
}

// byte -> (value of low nibble, value of high nibble) * 2^-14 as float2
__device__ __forceinline__ float2 sw_fp4_pair(unsigned b) {
    const unsigned h = ((b & 0x8u) << 12) | ((b & 0x7u) << 9) | ((b & 0x80u) << 24) | ((b & 0x70u) << 21);
    return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}

// sum over one 16-byte piece: 32 columns of x times the 32 codes, times 2^-14
__device__ __forceinline__ float sw_fp4_piece(const uint4 w, const float4 *xs, int) {
    // four partial sums (one per 8 columns): one chain of 32 dependent multiply-adds per piece would leave the warp
    // waiting on arithmetic latency
    float p[4];
    const unsigned ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const float4 xa = __ldg(xs + 2 * q), xb = __ldg(xs + 2 * q + 1);      // columns 8q .. 8q+7
        const float2 v0 = sw_fp4_pair(ww[q] & 0xFFu), v1 = sw_fp4_pair((ww[q] >> 8) & 0xFFu);
        const float2 v2 = sw_fp4_pair((ww[q] >> 16) & 0xFFu), v3 = sw_fp4_pair(ww[q] >> 24);
        float a = xa.x * v0.x, b = xa.y * v0.y;
        a = fmaf(xa.z, v1.x, a); b = fmaf(xa.w, v1.y, b);
        a = fmaf(xb.x, v2.x, a); b = fmaf(xb.y, v2.y, b);
        a = fmaf(xb.z, v3.x, a); b = fmaf(xb.w, v3.y, b);
        p[q] = a + b;
    }
    return (p[0] + p[1]) + (p[2] + p[3]);
}

// GLU = false: Y[z, o] = X[z, :] . W[o, :]                       (z = blockIdx.y: a token row, or an expert slot)
// GLU = true : Y[z, o] = silu(min(g, lim)) * clamp(u, -lim, lim), g = X . W[o, :], u = X . W[O + o, :]
// sel != nullptr: slot z uses the rows of expert sel[z] (weights at e * rows_per_expert).
template <bool GLU>
__global__ void __launch_bounds__(SW_FP4_WARPS * 32)
k_fp4_rows(const uint8_t *__restrict__ P, const uint8_t *__restrict__ ES, const int *__restrict__ sel, long long rows_per_expert,
           const float *__restrict__ X, long long x_stride, float *__restrict__ Y, long long y_stride,
           int I, int O, float limit) {
    // The token row (16 KB at most per warp step) is read straight through L1: every warp of the CTA reads the same
    // pieces, so after the first touch they are hits, and no CTA waits for a staging copy before it streams weights.
    const int z = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float4 *sw_fp4_x = reinterpret_cast<const float4 *>(X + (size_t)z * x_stride);
    const long long erow = sel ? (long long)sel[z] * rows_per_expert : 0;
    constexpr int RW = SW_FP4_RW(GLU);
    const int o0 = (blockIdx.x * SW_FP4_WARPS + warp) * RW;
    if (o0 >= O) return;
    constexpr int NR = GLU ? 2 * RW : RW;                          // weight rows per warp
    const uint8_t *pw[NR], *pe[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const int o = min(o0 + (r % RW), O - 1) + (GLU && r >= RW ? O : 0);
        pw[r] = P + (size_t)(erow + o) * (I / 2);
        pe[r] = ES + (size_t)(erow + o) * (I / 32);
    }
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r] = 0.f;
    const int nblk = I / 32;
    // software pipeline: the pieces of the next step are requested before the current ones are multiplied
    uint4 w[NR]; unsigned e[NR];
    if (lane < nblk) {
#pragma unroll
        for (int r = 0; r < NR; r++) { w[r] = reinterpret_cast<const uint4 *>(pw[r])[lane]; e[r] = pe[r][lane]; }
    }
    for (int b = lane; b < nblk; b += 32) {
        uint4 wn[NR]; unsigned en[NR];
        const bool more = b + 32 < nblk;
        if (more) {
#pragma unroll
            for (int r = 0; r < NR; r++) { wn[r] = reinterpret_cast<const uint4 *>(pw[r])[b + 32]; en[r] = pe[r][b + 32]; }
        }
        const float4 *xs = sw_fp4_x + b * 8;
#pragma unroll
        for (int r = 0; r < NR; r++) acc[r] = fmaf(sw_fp4_piece(w[r], xs, b & 7) * 16384.f, sw_ue8m0(e[r]), acc[r]);
        if (more) {
#pragma unroll
            for (int r = 0; r < NR; r++) { w[r] = wn[r]; e[r] = en[r]; }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; r++)
#pragma unroll
        for (int off = 16; off; off >>= 1) acc[r] += __shfl_xor_sync(SW_FULL_MASK, acc[r], off);
    if (lane == 0) {
        float *y = Y + (size_t)z * y_stride;
#pragma unroll
        for (int r = 0; r < RW; r++) {
            if (o0 + r >= O) break;
            if (GLU) {
                float g = acc[r], u = acc[RW + r];
                g = g > limit ? limit : g;
                u = u > limit ? limit : (u < -limit ? -limit : u);
                y[o0 + r] = (g / (1.f + expf(-g))) * u;
            } else {
                y[o0 + r] = acc[r];
            }
        }
    }
}

// out[i] = sum_k fma(w[k], part[k, i]) in the order given (the reference's axpy chain)
__global__ void __launch_bounds__(256)
k_fp4_combine(const float *__restrict__ part, const float *__restrict__ w, int K, int D, float *__restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= D) return;
    float a = 0.f;
    for (int k = 0; k < K; k++) a = fmaf(w[k], part[(size_t)k * D + i], a);
    out[i] = a;
}

static int sw_fp4_launch(const SwLaunchCfg &c, bool glu, const void *P, const void *ES, const int *sel, long long rows_per_expert,
                         const float *X, long long x_stride, float *Y, long long y_stride, int Z, int I, int O, float limit) {
    if (Z <= 0 || O <= 0) return 0;
    if (I <= 0 || (I % 32) || (((uintptr_t)P) & 15) || ((I / 2) % 16)) return -1;
    const size_t smem = 0;
    static SwPerDevice attr_done;
    if (attr_done.get(c.dev, [] {
            if (cudaFuncSetAttribute(k_fp4_rows<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
                cudaFuncSetAttribute(k_fp4_rows<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) { cudaGetLastError(); return -1; }
            return 1; }) <= 0) return -1;
    const int per_cta = SW_FP4_WARPS * (glu ? SW_FP4_RW(true) : SW_FP4_RW(false));
    dim3 grid((unsigned)((O + per_cta - 1) / per_cta), (unsigned)Z);
    if (glu) k_fp4_rows<true><<<grid, SW_FP4_WARPS * 32, smem, c.stream>>>((const uint8_t *)P, (const uint8_t *)ES, sel, rows_per_expert, X, x_stride, Y, y_stride, I, O, limit);
    else k_fp4_rows<false><<<grid, SW_FP4_WARPS * 32, smem, c.stream>>>((const uint8_t *)P, (const uint8_t *)ES, sel, rows_per_expert, X, x_stride, Y, y_stride, I, O, limit);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// y[S,O] = x[S,I] * dequant(P, ES)^T
int sw_launch_fp4_rows(const SwLaunchCfg &c, const float *x, const void *P, const void *ES, float *y, int S, int I, int O) {
    return sw_fp4_launch(c, false, P, ES, nullptr, 0, x, I, y, O, S, I, O, 0.f);
}

// out[D] = sum_k w[k] * down_k(glu_k(x)) for the K experts sel[k] (device arrays), glu [K, I] and part [K, D] scratch
int sw_launch_fp4_experts(const SwLaunchCfg &c, const float *x, const void *gu_q, const void *gu_es, const void *dn_q,
                          const void *dn_es, const int *sel, const float *w, int K, int I, int D, float limit,
                          float *glu, float *part, float *out) {
    if (K <= 0) return cudaMemsetAsync(out, 0, (size_t)D * 4, c.stream) == cudaSuccess ? 0 : -1;
    if (sw_fp4_launch(c, true, gu_q, gu_es, sel, 2LL * I, x, 0, glu, I, K, D, I, limit)) return -1;
    if (sw_fp4_launch(c, false, dn_q, dn_es, sel, D, glu, I, part, D, K, I, D, 0.f)) return -1;
    k_fp4_combine<<<(unsigned)((D + 255) / 256), 256, 0, c.stream>>>(part, w, K, D, out);
    sw_count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
