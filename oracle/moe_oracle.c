/* moe_oracle.c -- CPU restatement of sabrewing's MoE-block hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against (tests, the smoke check, and the timed CPU baseline of the bench).  The
 * shipped library never links, loads or calls it.
 *
 * Parity pin: every function below is compared bit-for-bit (exact mode) against
 * the reference's own code compiled from its sources (see ref_shim.c / Makefile in
 * this directory), against the reference tests' hand-computed nibble vectors
 * (c/tests/test_backend_cuda.cu:105-110) and against committed golden fixtures.
 *
 * Each function cites the reference file:line it restates.  "exact" means the
 * reference's double-accumulate contract (what its token-exact model oracle
 * validates, c/laguna.c:1910); exact=0 is a plain float-accumulate port used only
 * as a fallback timing arm when the compiled reference is unavailable.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

enum { ORC_ROUTE_SIGMOID = 0, ORC_ROUTE_SOFTMAX = 1,     /* c/moe_arch.h:22 */
       ORC_ROUTE_SOFTPLUS = 2 };                          /* softplusf (c/moe_math.h:54) as the gate; no reference router uses it */
enum { ORC_SHARED_NONE = 0, ORC_SHARED_UNSCALED = 1 };   /* c/moe_arch.h:25-30 */

/* One MoE layer over plain arrays.  Field meaning follows MoeDesc
 * (c/moe_arch.h:33-41) plus the Laguna int4 container (c/laguna.c:92-96,415-419):
 * gate_up rows of expert e start at row e*2I (gate rows, then up rows), down rows
 * at e*D. */
typedef struct {
    int D, I, SI, E, K;
    int route_act, use_corr_bias, norm_topk;
    float route_scale;
    int shared_mode;
    int gs;                       /* 0 = one scale per row (moe_quant.h); >0 = per-group scales (quant.h fmt=4) */
    const float *router_w;        /* [E,D] f32 */
    const float *corr_bias;       /* [E] or NULL */
    const float *logit_bias;      /* [E] or NULL; added to router logits before the gate activation */
    const uint8_t *gu_q; const float *gu_s;   /* [E*2I, D/2], scales [E*2I] or [E*2I, ceil(D/gs)] */
    const uint8_t *dn_q; const float *dn_s;   /* [E*D, I/2],  scales [E*D]  or [E*D, ceil(I/gs)]  */
    const uint16_t *sh_gate, *sh_up, *sh_down; /* bf16 [SI,D],[SI,D],[D,SI] */
} OrcLayer;

/* ---------------- scalar math (c/moe_math.h:51-72) ---------------- */
static inline float orc_bf16_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static inline float orc_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }   /* c/moe_math.h:54 */
static inline float orc_silu(float x) { return x / (1.f + expf(-x)); }          /* c/moe_math.h:53 */

/* c/moe_math.h:58-62 */
ORC_API void orc_rmsnorm_rows(float *out, const float *x, const float *w, int S, int D, float eps) {
    for (int s = 0; s < S; s++) {
        const float *xr = x + (int64_t)s * D; float *o = out + (int64_t)s * D;
        double ss = 0; for (int i = 0; i < D; i++) ss += (double)xr[i] * xr[i];
        float inv = 1.f / sqrtf((float)(ss / D) + eps);
        for (int i = 0; i < D; i++) o[i] = xr[i] * inv * (w ? w[i] : 1.f);
    }
}

/* c/moe_math.h:68-72: float max, float expf, DOUBLE running sum, reciprocal multiply */
ORC_API void orc_softmax_row(float *x, int n) {
    float mx = x[0]; for (int i = 1; i < n; i++) if (x[i] > mx) mx = x[i];
    double s = 0; for (int i = 0; i < n; i++) { x[i] = expf(x[i] - mx); s += x[i]; }
    float inv = (float)(1.0 / s); for (int i = 0; i < n; i++) x[i] *= inv;
}

/* ---------------- quantiser (c/tools/kernel_check.c:27-35) ---------------- */
ORC_API void orc_quant_rows_i4(const float *w, int rows, int I, uint8_t *packed, float *scale) {
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const float *wr = w + (int64_t)r * I; uint8_t *p = packed + (int64_t)r * (I / 2);
        float mx = 0; for (int i = 0; i < I; i++) { float a = fabsf(wr[i]); if (a > mx) mx = a; }
        float s = mx / 7.f; if (s < 1e-12f) s = 1e-12f; scale[r] = s;
        for (int c = 0; c < I / 2; c++) {
            int lo = (int)lrintf(wr[2 * c] / s);     if (lo < -8) lo = -8; if (lo > 7) lo = 7;
            int hi = (int)lrintf(wr[2 * c + 1] / s); if (hi < -8) hi = -8; if (hi > 7) hi = 7;
            p[c] = (uint8_t)((lo + 8) | ((hi + 8) << 4));
        }
    }
}

/* ---------------- GEMMs ---------------- */
/* y[S,O] = x[S,I] . W[O,I]^T, f32 weights (c/moe_matmul.h:25-55). */
ORC_API void orc_matmul_f32(float *y, const float *x, const float *W, int S, int I, int O, int exact) {
    #pragma omp parallel for schedule(static) if ((int64_t)S * O >= 512)
    for (int o = 0; o < O; o++) {
        const float *w = W + (int64_t)o * I;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            if (exact) { double sm = 0; for (int i = 0; i < I; i++) sm += (double)xs[i] * w[i]; y[(int64_t)s * O + o] = (float)sm; }
            else       { float sm = 0;  for (int i = 0; i < I; i++) sm += xs[i] * w[i];          y[(int64_t)s * O + o] = sm; }
        }
    }
}

/* bf16 weights expanded exactly, f32 activations (round_x=0 contract, c/moe_matmul.h:65,92-121). */
ORC_API void orc_matmul_bf16(float *y, const float *x, const uint16_t *W, int S, int I, int O, int exact) {
    #pragma omp parallel for schedule(static) if ((int64_t)S * O >= 512)
    for (int o = 0; o < O; o++) {
        const uint16_t *w = W + (int64_t)o * I;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            if (exact) { double sm = 0; for (int i = 0; i < I; i++) sm += (double)xs[i] * orc_bf16_f32(w[i]); y[(int64_t)s * O + o] = (float)sm; }
            else       { float sm = 0;  for (int i = 0; i < I; i++) sm += xs[i] * orc_bf16_f32(w[i]);          y[(int64_t)s * O + o] = sm; }
        }
    }
}

/* int4, one f32 scale per output row: value = nibble-8, low nibble = even column
 * (c/moe_quant.h:45-125 for S=1, :138-217 batched; every (s,o) reduces alone). */
ORC_API void orc_matmul_q4(float *y, const float *x, const uint8_t *packed, const float *scale,
                           int S, int I, int O, int exact) {
    #pragma omp parallel for schedule(static) if ((int64_t)S * O >= 512)
    for (int o = 0; o < O; o++) {
        const uint8_t *p = packed + (int64_t)o * (I / 2);
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            if (exact) {
                double a = 0;
                for (int c = 0; c < I / 2; c++) {
                    uint8_t b = p[c];
                    a += (double)xs[2 * c] * ((int)(b & 0xF) - 8) + (double)xs[2 * c + 1] * ((int)(b >> 4) - 8);
                }
                y[(int64_t)s * O + o] = (float)(a * scale[o]);
            } else {
                float a = 0;
                for (int c = 0; c < I / 2; c++) {
                    uint8_t b = p[c];
                    a += xs[2 * c] * ((int)(b & 0xF) - 8) + xs[2 * c + 1] * ((int)(b >> 4) - 8);
                }
                y[(int64_t)s * O + o] = a * scale[o];
            }
        }
    }
}

/* fp4: e2m1 codes, two per byte (low nibble = even column), one ue8m0 exponent byte per 32 input
 * columns: value = lut[nibble] * 2^(es[o, col/32] - 127)  (c/moe_quant.h:219-257). */
static const float orc_fp4_lut[16] = { 0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                       -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f };
/* 0xFF (the format's NaN) decodes to 0, 0 to the denormal 2^-127 (c/moe_quant.h:250-256). */
static inline float orc_ue8m0(uint8_t e) {
    if (e == 0xFF) return 0.f;
    if (e == 0) return 5.8774717541114375e-39f;
    uint32_t u = (uint32_t)e << 23; float f; memcpy(&f, &u, 4); return f;
}
/* y[S,O] = x[S,I] * dequant(packed, es)^T.  exact: the double-accumulate loop of
 * c/moe_quant.h:289-301 (per byte: (x0*lut0 + x1*lut1) * scale, added in column order);
 * exact=0: a plain float port with one partial sum per 32-column block. */
ORC_API void orc_matmul_fp4(float *y, const float *x, const uint8_t *packed, const uint8_t *es,
                            int S, int I, int O, int exact) {
    #pragma omp parallel for schedule(static) if ((int64_t)S * O >= 512)
    for (int o = 0; o < O; o++) {
        const uint8_t *p = packed + (int64_t)o * (I / 2);
        const uint8_t *e = es + (int64_t)o * (I / 32);
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            if (exact) {
                double a = 0;
                for (int c = 0; c < I / 2; c++) {
                    uint8_t b = p[c];
                    double sc = orc_ue8m0(e[(2 * c) / 32]);
                    a += ((double)xs[2 * c] * orc_fp4_lut[b & 0xF] + (double)xs[2 * c + 1] * orc_fp4_lut[b >> 4]) * sc;
                }
                y[(int64_t)s * O + o] = (float)a;
            } else {
                float a = 0;
                for (int blk = 0; blk < I / 32; blk++) {
                    float part = 0, sc = orc_ue8m0(e[blk]);
                    for (int c = blk * 16; c < blk * 16 + 16; c++) {
                        uint8_t b = p[c];
                        part += xs[2 * c] * orc_fp4_lut[b & 0xF] + xs[2 * c + 1] * orc_fp4_lut[b >> 4];
                    }
                    a += part * sc;
                }
                y[(int64_t)s * O + o] = a;
            }
        }
    }
}

/* K routed fp4 experts of one token, DeepSeek-V4's clamped SwiGLU (c/deepseek.c:820-842):
 * gate clamped from above at limit, up clamped to [-limit, limit]; the experts' outputs are
 * added as out += w[a]*y_a in the order given (c/deepseek.c:1571, c/backend_cuda_laguna.cu:389-395).
 * h: scratch of 2*I + D floats. */
ORC_API void orc_experts_fp4(float *out, const float *x, const uint8_t *gu_q, const uint8_t *gu_es,
                             const uint8_t *dn_q, const uint8_t *dn_es, const int *sel, const float *w,
                             int K, int I, int D, float limit, int exact, float *h) {
    float *g = h, *u = h + I, *tmp = h + 2 * I;
    for (int i = 0; i < D; i++) out[i] = 0.f;
    for (int a = 0; a < K; a++) {
        const int64_t e = sel[a];
        orc_matmul_fp4(g, x, gu_q + e * 2 * I * (D / 2), gu_es + e * 2 * I * (D / 32), 1, D, 2 * I, exact);
        for (int i = 0; i < I; i++) {
            float gi = g[i] > limit ? limit : g[i];
            float ui = u[i] > limit ? limit : (u[i] < -limit ? -limit : u[i]);
            g[i] = orc_silu(gi) * ui;
        }
        orc_matmul_fp4(tmp, g, dn_q + e * D * (I / 2), dn_es + e * D * (I / 32), 1, I, D, exact);
        for (int i = 0; i < D; i++) out[i] += w[a] * tmp[i];
    }
}

/* int4 with one scale per gs inputs: y = sum_g scale[o,g] * sum_{i in g} x_i*(nib_i-8)
 * (c/quant.h:167-202; double form follows the plain reference in
 * c/tests/test_i4_grouped.c:30-54, which multiplies the scale into every term). */
ORC_API void orc_matmul_i4_grouped(float *y, const float *x, const uint8_t *q4, const float *scale,
                                   int S, int I, int O, int gs, int exact) {
    int rb = (I + 1) / 2, ng = (I + gs - 1) / gs;
    #pragma omp parallel for schedule(static) if ((int64_t)S * O >= 512)
    for (int o = 0; o < O; o++) {
        const uint8_t *w = q4 + (int64_t)o * rb; const float *scl = scale + (int64_t)o * ng;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (int64_t)s * I;
            if (exact) {
                double a = 0;
                for (int i = 0; i < I; i++) {
                    uint8_t b = w[i >> 1]; int nib = (i & 1) ? (int)(b >> 4) : (int)(b & 0xF);
                    a += (double)xs[i] * (double)(nib - 8) * (double)scl[i / gs];
                }
                y[(int64_t)s * O + o] = (float)a;
            } else {
                float a = 0;
                for (int g = 0; g * gs < I; g++) {
                    int base = g * gs, end = base + gs < I ? base + gs : I; float part = 0;
                    for (int i = base; i < end; i++) {
                        uint8_t b = w[i >> 1]; int nib = (i & 1) ? (int)(b >> 4) : (int)(b & 0xF);
                        part += xs[i] * (float)(nib - 8);
                    }
                    a += part * scl[g];
                }
                y[(int64_t)s * O + o] = a;
            }
        }
    }
}

static void orc_expert_mm(const OrcLayer *L, float *y, const float *x, const uint8_t *q, const float *s,
                          int64_t row0, int S, int I, int O, int exact) {
    if (L->gs > 0) {
        int ng = (I + L->gs - 1) / L->gs;
        orc_matmul_i4_grouped(y, x, q + row0 * ((I + 1) / 2), s + row0 * ng, S, I, O, L->gs, exact);
    } else {
        orc_matmul_q4(y, x, q + row0 * (I / 2), s + row0, S, I, O, exact);
    }
}

/* ---------------- routing ---------------- */
/* c/moe_arch.h:64-89: K rounds of arg-max over score+bias, strict >, ascending scan
 * (ties to the lower id); if nothing beats -1e30f (all non-finite) take the lowest
 * unselected id. */
ORC_API void orc_topk(const float *score, const float *corr_bias, int use_bias, int E, int K, int *sel) {
    for (int a = 0; a < K; a++) {
        int best = -1; float bv = -1e30f;
        for (int e = 0; e < E; e++) {
            int used = 0; for (int b = 0; b < a; b++) if (sel[b] == e) { used = 1; break; }
            if (used) continue;
            float s = score[e] + (use_bias && corr_bias ? corr_bias[e] : 0.f);
            if (s > bv) { bv = s; best = e; }
        }
        if (best < 0) {
            for (int e = 0; e < E && best < 0; e++) {
                int used = 0; for (int b = 0; b < a; b++) if (sel[b] == e) { used = 1; break; }
                if (!used) best = e;
            }
            if (best < 0) best = 0;
        }
        sel[a] = best;
    }
}

/* Router logits -> gate activation -> top-k -> combine weights for S rows
 * (c/moe_block.h:24-31; batched form c/laguna.c:698-706).  scores[S,E] optional. */
ORC_API void orc_route(const OrcLayer *L, const float *x, int S, int exact,
                       int *sel, float *w, float *scores_out) {
    int E = L->E, K = L->K, D = L->D;
    float *rl = (float*)malloc((size_t)S * E * sizeof(float));
    orc_matmul_f32(rl, x, L->router_w, S, D, E, exact);
    for (int s = 0; s < S; s++) {
        float *r = rl + (int64_t)s * E;
        if (L->logit_bias) for (int e = 0; e < E; e++) r[e] += L->logit_bias[e];
        if (L->route_act == ORC_ROUTE_SOFTMAX) orc_softmax_row(r, E);
        else if (L->route_act == ORC_ROUTE_SOFTPLUS) for (int e = 0; e < E; e++) r[e] = orc_softplus(r[e]);
        else for (int e = 0; e < E; e++) r[e] = 1.f / (1.f + expf(-r[e]));
        int *sl = sel + (int64_t)s * K; float *wr = w + (int64_t)s * K;
        orc_topk(r, L->corr_bias, L->use_corr_bias, E, K, sl);
        for (int a = 0; a < K; a++) wr[a] = r[sl[a]];
        if (L->norm_topk) { float sm = 0; for (int a = 0; a < K; a++) sm += wr[a]; for (int a = 0; a < K; a++) wr[a] /= sm; }
    }
    if (scores_out) memcpy(scores_out, rl, (size_t)S * E * sizeof(float));
    free(rl);
}

/* Counting sort of the S*K (row, expert) pairs by expert (c/laguna.c:709-723):
 * groups in ascending expert id, empty experts skipped, pairs inside a group in
 * ascending flat index s*K+a.  Returns G. */
ORC_API int orc_group(const int *sel, int S, int K, int E,
                      int *gexp, int *gbeg, int *gcnt, int *grow, int *rowof) {
    int T = S * K;
    int *cnt = (int*)calloc((size_t)E, sizeof(int)), *pos = (int*)malloc((size_t)E * sizeof(int));
    for (int i = 0; i < T; i++) cnt[sel[i]]++;
    int G = 0, off = 0;
    for (int e = 0; e < E; e++) {
        if (!cnt[e]) continue;
        gexp[G] = e; gbeg[G] = off; gcnt[G] = cnt[e]; pos[e] = off; off += cnt[e]; G++;
    }
    for (int s = 0; s < S; s++) for (int a = 0; a < K; a++) {
        int slot = pos[sel[s * K + a]]++;
        grow[slot] = s; rowof[s * K + a] = slot;
    }
    free(cnt); free(pos);
    return G;
}

/* ---------------- experts ---------------- */
/* One routed expert over n rows: gate_up -> silu*up -> down (c/laguna.c:577-588,745-752). */
static void orc_expert_rows(const OrcLayer *L, int e, const float *xg, int n, float *gu, float *glu,
                            float *out, int exact) {
    int D = L->D, I = L->I;
    orc_expert_mm(L, gu, xg, L->gu_q, L->gu_s, (int64_t)e * 2 * I, n, D, 2 * I, exact);
    for (int j = 0; j < n; j++) {
        const float *gr = gu + (int64_t)j * 2 * I; float *o = glu + (int64_t)j * I;
        for (int i = 0; i < I; i++) o[i] = orc_silu(gr[i]) * gr[I + i];
    }
    orc_expert_mm(L, out, glu, L->dn_q, L->dn_s, (int64_t)e * D, n, I, D, exact);
}

/* Shared expert over S rows (c/laguna.c:596-602 per token, :777-781 batched). */
ORC_API void orc_shared_rows(const OrcLayer *L, const float *x, int S, float *so, int exact) {
    int D = L->D, SI = L->SI;
    float *sg = (float*)malloc((size_t)S * SI * sizeof(float)), *su = (float*)malloc((size_t)S * SI * sizeof(float));
    orc_matmul_bf16(sg, x, L->sh_gate, S, D, SI, exact);
    orc_matmul_bf16(su, x, L->sh_up, S, D, SI, exact);
    for (int64_t i = 0; i < (int64_t)S * SI; i++) sg[i] = orc_silu(sg[i]) * su[i];
    orc_matmul_bf16(so, sg, L->sh_down, S, SI, D, exact);
    free(sg); free(su);
}

/* hout[S,D] += MoE(x[S,D]), one token at a time (c/moe_block.h:18-54 driven as in
 * c/laguna.c:818-821).  The weighted sum is accumulated in rank order with the
 * multiply-add the reference's build contracts to an FMA. */
ORC_API void orc_moe_rows(const OrcLayer *L, const float *x, float *hout, int S, int exact) {
    int D = L->D, I = L->I, K = L->K;
    int *sel = (int*)malloc((size_t)S * K * sizeof(int)); float *w = (float*)malloc((size_t)S * K * sizeof(float));
    orc_route(L, x, S, exact, sel, w, NULL);
    float *gu = (float*)malloc((size_t)2 * I * sizeof(float)), *glu = (float*)malloc((size_t)I * sizeof(float));
    float *scr = (float*)malloc((size_t)D * sizeof(float)), *acc = (float*)malloc((size_t)D * sizeof(float));
    for (int s = 0; s < S; s++) {
        const float *xs = x + (int64_t)s * D; float *o = hout + (int64_t)s * D;
        for (int i = 0; i < D; i++) acc[i] = 0;
        for (int a = 0; a < K; a++) {
            orc_expert_rows(L, sel[s * K + a], xs, 1, gu, glu, scr, exact);
            float wa = w[s * K + a];
            for (int i = 0; i < D; i++) acc[i] = fmaf(wa, scr[i], acc[i]);
        }
        for (int i = 0; i < D; i++) acc[i] *= L->route_scale;
        if (L->shared_mode != ORC_SHARED_NONE) {
            orc_shared_rows(L, xs, 1, scr, exact);
            for (int i = 0; i < D; i++) acc[i] += scr[i];
        }
        for (int i = 0; i < D; i++) o[i] += acc[i];
    }
    free(sel); free(w); free(gu); free(glu); free(scr); free(acc);
}

/* hout[S,D] += MoE(x[S,D]) grouped by expert (c/laguna.c:689-787).  Optional
 * outputs (may be NULL): sel/w [S*K], G, gexp/gbeg/gcnt [E], grow/rowof [S*K],
 * routed [S,D] = the unscaled weighted routed sum (what lag_cuda_moe_group
 * returns, c/backend_cuda_laguna.h:52-75). */
ORC_API void orc_moe_group(const OrcLayer *L, const float *x, float *hout, int S, int exact,
                           int *sel_o, float *w_o, int *G_o, int *gexp_o, int *gbeg_o, int *gcnt_o,
                           int *grow_o, int *rowof_o, float *routed_o) {
    int D = L->D, I = L->I, E = L->E, K = L->K, T = S * K;
    int *sel = (int*)malloc((size_t)T * sizeof(int)); float *w = (float*)malloc((size_t)T * sizeof(float));
    orc_route(L, x, S, exact, sel, w, NULL);
    int *gexp = (int*)malloc((size_t)E * sizeof(int)), *gbeg = (int*)malloc((size_t)E * sizeof(int));
    int *gcnt = (int*)malloc((size_t)E * sizeof(int));
    int *grow = (int*)malloc((size_t)T * sizeof(int)), *rowof = (int*)malloc((size_t)T * sizeof(int));
    int G = orc_group(sel, S, K, E, gexp, gbeg, gcnt, grow, rowof);

    float *slots = (float*)malloc((size_t)T * D * sizeof(float));
    int maxn = 0; for (int g = 0; g < G; g++) if (gcnt[g] > maxn) maxn = gcnt[g];
    float *xg = (float*)malloc((size_t)maxn * D * sizeof(float));
    float *gu = (float*)malloc((size_t)maxn * 2 * I * sizeof(float)), *glu = (float*)malloc((size_t)maxn * I * sizeof(float));
    for (int g = 0; g < G; g++) {
        int e = gexp[g], n = gcnt[g], beg = gbeg[g];
        for (int j = 0; j < n; j++) memcpy(xg + (int64_t)j * D, x + (int64_t)grow[beg + j] * D, (size_t)D * sizeof(float));
        orc_expert_rows(L, e, xg, n, gu, glu, slots + (int64_t)beg * D, exact);
    }
    float *acc = (float*)malloc((size_t)S * D * sizeof(float));
    for (int s = 0; s < S; s++) {
        float *o = acc + (int64_t)s * D;
        for (int i = 0; i < D; i++) o[i] = 0;
        for (int a = 0; a < K; a++) {
            const float *v = slots + (int64_t)rowof[s * K + a] * D; float wa = w[s * K + a];
            for (int i = 0; i < D; i++) o[i] = fmaf(wa, v[i], o[i]);
        }
    }
    if (routed_o) memcpy(routed_o, acc, (size_t)S * D * sizeof(float));
    for (int64_t i = 0; i < (int64_t)S * D; i++) acc[i] *= L->route_scale;
    if (L->shared_mode != ORC_SHARED_NONE) {
        float *so = (float*)malloc((size_t)S * D * sizeof(float));
        orc_shared_rows(L, x, S, so, exact);
        for (int64_t i = 0; i < (int64_t)S * D; i++) hout[i] += acc[i] + so[i];
        free(so);
    } else {
        for (int64_t i = 0; i < (int64_t)S * D; i++) hout[i] += acc[i];
    }
    if (sel_o) memcpy(sel_o, sel, (size_t)T * sizeof(int));
    if (w_o) memcpy(w_o, w, (size_t)T * sizeof(float));
    if (G_o) *G_o = G;
    if (gexp_o) memcpy(gexp_o, gexp, (size_t)G * sizeof(int));
    if (gbeg_o) memcpy(gbeg_o, gbeg, (size_t)G * sizeof(int));
    if (gcnt_o) memcpy(gcnt_o, gcnt, (size_t)G * sizeof(int));
    if (grow_o) memcpy(grow_o, grow, (size_t)T * sizeof(int));
    if (rowof_o) memcpy(rowof_o, rowof, (size_t)T * sizeof(int));
    free(sel); free(w); free(gexp); free(gbeg); free(gcnt); free(grow); free(rowof);
    free(slots); free(xg); free(gu); free(glu); free(acc);
}

/* Weighted routed sum for given routing: the CPU twin of the two reference GPU
 * entry points (c/backend_cuda_laguna.cu:240-281 for one row, :495-546 grouped). */
ORC_API void orc_experts_given_routing(const OrcLayer *L, const float *x, int S, const int *sel, const float *w,
                                       float *routed, int exact) {
    int D = L->D, I = L->I, K = L->K;
    float *gu = (float*)malloc((size_t)2 * I * sizeof(float)), *glu = (float*)malloc((size_t)I * sizeof(float));
    float *scr = (float*)malloc((size_t)D * sizeof(float));
    for (int s = 0; s < S; s++) {
        float *o = routed + (int64_t)s * D;
        for (int i = 0; i < D; i++) o[i] = 0;
        for (int a = 0; a < K; a++) {
            orc_expert_rows(L, sel[s * K + a], x + (int64_t)s * D, 1, gu, glu, scr, exact);
            float wa = w[s * K + a];
            for (int i = 0; i < D; i++) o[i] = fmaf(wa, scr[i], o[i]);
        }
    }
    free(gu); free(glu); free(scr);
}

ORC_API int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
