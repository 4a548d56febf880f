/* ref_shim.c -- thin export layer over the UNMODIFIED reference sources.
 *
 * TEST INFRASTRUCTURE ONLY.  This translation unit #includes the reference's own
 * c/laguna.c (its main renamed) from where the reference checkout lies, so the
 * functions exported here run the reference's real lag_moe_rows / lag_moe_group /
 * moe_block / matmul_* code.  Nothing from the reference is copied into this
 * repository; the Makefile beside this file passes -I<reference>/c.  It is used to
 * validate the restatement in moe_oracle.c, to generate golden fixtures, and as
 * the timed CPU baseline ("kind": "reference").
 */
#define main laguna_main_unused
#include "laguna.c"
#undef main

#define REF_API __attribute__((visibility("default")))

/* Same layout as OrcLayer in moe_oracle.c. */
typedef struct {
    int D, I, SI, E, K;
    int route_act, use_corr_bias, norm_topk;
    float route_scale;
    int shared_mode;
    int gs;
    const float *router_w;
    const float *corr_bias;
    const float *logit_bias;
    const uint8_t *gu_q; const float *gu_s;
    const uint8_t *dn_q; const float *dn_s;
    const uint16_t *sh_gate, *sh_up, *sh_down;
} RefLayer;

static void ref_fill(const RefLayer *r, Model *m, Layer *L) {
    memset(m, 0, sizeof *m); memset(L, 0, sizeof *L);
    m->c.hidden = r->D; m->c.moe_inter = r->I; m->c.shared_inter = r->SI;
    m->c.n_experts = r->E; m->c.topk = r->K; m->c.norm_topk = r->norm_topk;
    m->c.route_scale = r->route_scale;
    m->xq = 1; m->res_dt = 1; m->L = L;
    L->router = (float*)r->router_w; L->ebias = (float*)r->corr_bias;
    L->gu_q = (uint8_t*)r->gu_q; L->gu_s = (float*)r->gu_s;
    L->dn_q = (uint8_t*)r->dn_q; L->dn_s = (float*)r->dn_s;
    L->sg = (void*)r->sh_gate; L->su = (void*)r->sh_up; L->sd = (void*)r->sh_down;
}

/* The reference's own Laguna MoE over S rows: lag_moe_rows (c/laguna.c:805-823),
 * i.e. lag_moe_group when group_on and S>1, else moe_block with the Laguna hooks.
 * Laguna semantics only: sigmoid gate, corr-bias selection, unscaled shared
 * expert, per-row-scale int4, no logit bias.  Returns -1 if the layer asks for
 * anything else. */
REF_API int ref_laguna_moe_rows(const RefLayer *r, const float *x, float *hout, int S, int exact, int group_on) {
    if (r->route_act != MOE_ROUTE_SIGMOID || r->shared_mode != MOE_SHARED_UNSCALED || r->gs != 0 ||
        r->logit_bias || (!r->use_corr_bias && r->corr_bias)) return -1;
    Model *m = malloc(sizeof *m); Layer *L = malloc(sizeof *L);
    ref_fill(r, m, L);
    g_exact = exact; g_res_dt = 1; g_group = group_on;
    lag_moe_rows(m, L, x, hout, S);
    free(m); free(L);
    return 0;
}

/* moe_block (c/moe_block.h:18-54) driven through hooks that call the reference's
 * kernels directly; covers softmax / no-shared / logit-bias layers that the
 * Laguna engine glue cannot express. */
typedef struct { const RefLayer *r; int exact; float *gu, *sg, *su; } HookCtx;
static void hk_router(void *cx, const float *x, float *lg) {
    HookCtx *c = cx; const RefLayer *r = c->r;
    matmul_f32(lg, x, r->router_w, 1, r->D, r->E, c->exact);
    if (r->logit_bias) for (int e = 0; e < r->E; e++) lg[e] += r->logit_bias[e];
}
static void hk_expert(void *cx, int e, const float *x, float *out) {
    HookCtx *c = cx; const RefLayer *r = c->r; int I = r->I, D = r->D;
    matmul_q4_k(c->gu, x, r->gu_q + (int64_t)(e * 2 * I) * (D / 2), r->gu_s + (int64_t)e * 2 * I, D, 2 * I, MOE_Q4_F32, c->exact);
    for (int i = 0; i < I; i++) c->gu[i] = siluf(c->gu[i]) * c->gu[I + i];
    matmul_q4_k(out, c->gu, r->dn_q + (int64_t)(e * D) * (I / 2), r->dn_s + (int64_t)e * D, I, D, MOE_Q4_F32, c->exact);
}
static void hk_shared(void *cx, const float *x, float *out) {
    HookCtx *c = cx; const RefLayer *r = c->r; int SI = r->SI, D = r->D;
    matmul_bf16_k(c->sg, x, r->sh_gate, 1, D, SI, 0, c->exact);
    matmul_bf16_k(c->su, x, r->sh_up, 1, D, SI, 0, c->exact);
    for (int i = 0; i < SI; i++) c->sg[i] = siluf(c->sg[i]) * c->su[i];
    matmul_bf16_k(out, c->sg, r->sh_down, 1, SI, D, 0, c->exact);
}
REF_API int ref_moe_block_rows(const RefLayer *r, const float *x, float *hout, int S, int exact) {
    if (r->gs != 0) return -1;
    HookCtx c = { r, exact, falloc(2 * r->I), falloc(r->SI > 0 ? r->SI : 1), falloc(r->SI > 0 ? r->SI : 1) };
    MoeDesc d = { r->E, r->K, (MoeRouteAct)r->route_act, r->use_corr_bias, r->norm_topk, r->route_scale,
                  (MoeSharedMode)r->shared_mode };
    MoeHooks h = { &c, hk_router, r->corr_bias, hk_expert, hk_shared, NULL };
    for (int s = 0; s < S; s++) moe_block(&d, &h, x + (int64_t)s * r->D, hout + (int64_t)s * r->D, r->D);
    free(c.gu); free(c.sg); free(c.su);
    return 0;
}

/* Kernel-level exports (signatures mirror moe_oracle.c). */
REF_API void ref_matmul_f32(float *y, const float *x, const float *W, int S, int I, int O, int exact) { matmul_f32(y, x, W, S, I, O, exact); }
REF_API void ref_matmul_bf16(float *y, const float *x, const uint16_t *W, int S, int I, int O, int exact) { matmul_bf16_k(y, x, W, S, I, O, 0, exact); }
REF_API void ref_matmul_q4(float *y, const float *x, const uint8_t *p, const float *sc, int S, int I, int O, int exact) { matmul_q4_kb(y, x, p, sc, S, I, O, MOE_Q4_F32, exact); }
REF_API void ref_matmul_fp4(float *y, const float *x, const uint8_t *p, const uint8_t *es, int S, int I, int O, int exact) { matmul_fp4_kb(y, x, p, es, S, I, O, exact); }
/* The K-expert loop of the reference's fp4 GPU self-test (c/deepseek.c:1557-1572), which is moe_row's
 * (c/deepseek.c:820-842), over the reference's own matmul_fp4_k and siluf.  h: 2*I + D floats. */
REF_API void ref_experts_fp4(float *out, const float *x, const uint8_t *gu, const uint8_t *gue, const uint8_t *dn,
                             const uint8_t *dne, const int *sel, const float *w, int K, int I, int D, float lim,
                             int exact, float *h) {
    float *g = h, *u = h + I, *tmp = h + 2 * I;
    for (int i = 0; i < D; i++) out[i] = 0;
    for (int a = 0; a < K; a++) {
        int e = sel[a];
        matmul_fp4_k(g, x, gu + (size_t)e * 2 * I * (D / 2), gue + (size_t)e * 2 * I * (D / 32), D, 2 * I, exact);
        for (int i = 0; i < I; i++) {
            float gi = g[i] > lim ? lim : g[i];
            float ui = u[i] > lim ? lim : (u[i] < -lim ? -lim : u[i]);
            g[i] = siluf(gi) * ui;
        }
        matmul_fp4_k(tmp, g, dn + (size_t)e * D * (I / 2), dne + (size_t)e * D * (I / 32), I, D, exact);
        for (int i = 0; i < D; i++) out[i] += w[a] * tmp[i];
    }
}
REF_API void ref_softmax_row(float *x, int n) { softmax_row(x, n); }
REF_API void ref_topk(const float *score, const float *bias, int use_bias, int E, int K, int *sel) { moe_topk(score, bias, use_bias, E, K, sel); }
REF_API void ref_rmsnorm_rows(float *out, const float *x, const float *w, int S, int D, float eps) {
    for (int s = 0; s < S; s++) rmsnorm_row(out + (int64_t)s * D, x + (int64_t)s * D, w, D, eps);
}
REF_API void ref_omp_autotune(void) { moe_omp_autotune(); }
REF_API int ref_physical_cores(void) { return moe_physical_cores(); }
REF_API int ref_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
REF_API void ref_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}
REF_API int ref_has_avx512(void) {
#if defined(__AVX512F__)
    return 1;
#else
    return 0;
#endif
}
