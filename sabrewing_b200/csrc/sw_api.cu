// C-ABI of the MoE-block backend: the lag_cuda_* drop-in tier and the
// descriptor-level sw_moe_* entry points (see include/sabrewing_b200.h).
#include "sw_common.cuh"
// the library is built with hidden visibility; only the C-ABI is exported
#pragma GCC visibility push(default)
#include "../../include/sabrewing_b200.h"
#pragma GCC visibility pop
#include <cuda_fp16.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>
#include <stdlib.h>

static std::atomic<long long> g_launches{0};
void sw_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long sw_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

std::mutex &sw_setup_mutex() { static std::mutex m; return m; }

static int sw_env_int(const char *name, int dflt) { const char *e = getenv(name); return e && *e ? atoi(e) : dflt; }
const SwTuning &sw_tuning() {
    static const SwTuning t = [] {
        SwTuning v{};
        v.expert_pref = 2;
        const char *e = getenv("SW_EXPERT_PATH");
        if (e && !strcmp(e, "umma")) v.expert_pref = 3;
        if (e && !strcmp(e, "tma")) v.expert_pref = 4;            // TMA decode kernels whatever the group size
        if (e && !strcmp(e, "mma")) v.expert_pref = 1;
        if (e && !strcmp(e, "simt")) v.expert_pref = 0;
        const char *f = getenv("SW_FORCE_SIMT");
        v.force_simt = (f && *f && *f != '0') ? 1 : 0;
        if (v.force_simt) v.expert_pref = 0;
        v.row_scale = sw_env_int("SW_ROW_SCALE", 1);
        v.umma_min_rows = sw_env_int("SW_UMMA_MIN_ROWS", 8);     // mean rows per group from which the tcgen05 kernels win (measured)
        v.tma_mt = sw_env_int("SW_TMA_MT", 0);
        if (v.tma_mt != 1 && v.tma_mt != 2) v.tma_mt = 0;
        v.tma_p = sw_env_int("SW_TMA_P", 0);
        v.mma_mt = sw_env_int("SW_MMA_MT", 0);
        v.fail_after = sw_env_int("SW_FAIL_AFTER", -1);
        return v;
    }();
    return t;
}

// Host-side failure injection, two hooks.
// (1) Compute calls, the reference's COLI_GPU_FAIL_AFTER (c/backend_cuda.cu:684-692): with SW_FAIL_AFTER=n in the
//     environment, or after sw_test_fail_after(n), every compute entry point reports failure once n calls have
//     succeeded (n = 0: every call fails); uploads, queries and context creation are not gated.  n < 0: off.
// (2) Allocations: after sw_test_fail_alloc(n) the n-th and every later device or page-locked allocation of this
//     library reports failure without calling CUDA (n <= 0: off).
static std::atomic<long> g_fail_after{-2}, g_calls{0};         // -2: not read from the environment yet
extern "C" void sw_test_fail_after(int n) { g_fail_after.store(n >= 0 ? n : -1); g_calls.store(0); }
static bool sw_fault_injected() {
    long n = g_fail_after.load(std::memory_order_relaxed);
    if (n == -2) { n = sw_tuning().fail_after; g_fail_after.store(n); }
    return n >= 0 && g_calls.fetch_add(1) >= n;
}
#define SW_GATE() do { if (sw_fault_injected()) return sw_fail("injected failure (SW_FAIL_AFTER)"); } while (0)
static std::atomic<int> g_fail_alloc{0}, g_alloc_count{0};
extern "C" void sw_test_fail_alloc(int n) { g_fail_alloc.store(n > 0 ? n : 0); g_alloc_count.store(0); }
static bool sw_inject_alloc_failure() {
    const int n = g_fail_alloc.load(std::memory_order_relaxed);
    return n > 0 && g_alloc_count.fetch_add(1) + 1 >= n;
}
static cudaError_t sw_malloc(void **p, size_t n) { if (sw_inject_alloc_failure()) { *p = nullptr; return cudaErrorMemoryAllocation; } return cudaMalloc(p, n); }
static cudaError_t sw_malloc_host(void **p, size_t n) { if (sw_inject_alloc_failure()) { *p = nullptr; return cudaErrorMemoryAllocation; } return cudaMallocHost(p, n); }

static thread_local char g_err[256] = "";
static int sw_fail(const char *fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof g_err, fmt, ap); va_end(ap);
    return -1;
}
extern "C" const char *sw_last_error(void) { return g_err; }
int sw_noalloc_fail(const char *msg) { return sw_fail("%s", msg); }
int sw_fail_text(const char *fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof g_err, fmt, ap); va_end(ap);
    return -1;
}

// A CUDA error is sticky only for faults; plain API failures (OOM, bad argument)
// are cleared so that the next call starts clean (the reference's hygiene rule,
// c/backend_cuda.cu:63-69).
static int sw_cuda_fail(cudaError_t e, const char *what) {
    cudaGetLastError();
    return sw_fail("%s: %s", what, cudaGetErrorString(e));
}
#define SW_CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return sw_cuda_fail(e_, #call); } while (0)

// grow-on-demand buffers (2x slack so size churn does not re-allocate every call)
struct SwBuf {
    void *p = nullptr; size_t cap = 0; bool pinned = false;
    int ensure(size_t need) {
        if (need <= cap) return 0;
        release();
        size_t want = need * 2;
        cudaError_t e = pinned ? sw_malloc_host(&p, want) : sw_malloc(&p, want);
        if (e != cudaSuccess) { p = nullptr; cap = 0; cudaGetLastError(); return -1; }
        cap = want; return 0;
    }
    void release() { if (p) { if (pinned) cudaFreeHost(p); else cudaFree(p); } p = nullptr; cap = 0; }
};

// scratch of the tcgen05 path: gathered fp16 hi/lo token rows [P, D] x2, chunk list
struct SwUmmaScratch { void *xg; int *nchunks; void *chunks; };

// ===========================================================================
// Descriptor-level context
// ===========================================================================
struct SwMoeCtx {
    int dev = 0, num_sms = 0;
    int maxT = 0, maxE = 0, maxK = 0, maxD = 0, maxI = 0, maxSI = 0;
    cudaStream_t stream = nullptr, last_stream = nullptr;
    cudaStream_t cpy = nullptr;              // forward_host: uploads the residual rows beside the kernels
    cudaEvent_t ev_res = nullptr; bool wait_res = false;   // set while a residual upload must precede the combine
    cudaStream_t aux = nullptr;                 // the shared expert runs here, beside routing and the routed experts
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_pack = nullptr;
    SwRouting r{};
    float *row_gate = nullptr;   // [T] weight of the shared expert per token (GATED / SIGMOID_GATED policies)
    float *glu = nullptr, *slots = nullptr, *sglu = nullptr, *so = nullptr, *routed = nullptr;
    float *dx = nullptr, *dout = nullptr, *hx = nullptr, *hout = nullptr;
    void *xp = nullptr;          // packed fp16 hi/lo copy of x for the tensor-core path
    SwUmmaScratch um{nullptr, nullptr, nullptr};
    double *rpart = nullptr;     // fp64 partial router logits [slices][T][E]
    void *spk = nullptr;         // packed bf16 hi/lo copy of x for the shared expert
    float *sums = nullptr;       // row sums of x and partial row sums of the SiLU*up rows
    int lastT = 0, lastK = 0, lastE = 0;
    int lastES = 0;              // row stride of the scores of the last routing (experts + the shared-pool logit, if any)
    int last_path = -1;          // expert kernels of the last experts/forward call (sw_moe_last_path)
    int umma_terms = 1;
    const float *row_back = nullptr;   // set by the last expert stage: per-token powers of two the combine step squares and applies (or null)
    int forced_path = -1;        // SW_OPT_EXPERT_PATH: -1 = choose by shape and group size          // fp16 terms per activation on the tcgen05 path: 1 = hi only, 2 = hi + lo
    int cap_on = 0, cap_prof = 0; long long cap_l0 = 0;   // open stage capture (sw_moe_capture_begin)
    // a shared-expert result left by sw_moe_shared for the next sw_moe_finish of the same row count
    int shared_T = -1, shared_slices = 1; float *shared_so = nullptr;
    void *block = nullptr;      // one device allocation holding all device scratch
    // optional per-stage CUDA-event timing (sw_moe_profile)
    int prof_on = 0, prof_calls = 0;
    cudaEvent_t *prof_ev = nullptr;   // [SW_PROF_MAX_CALLS][SW_NSTAGES+1]
};

// Layout of the `sums` scratch of the tensor-core paths: row sums of x [rows_x], the token rows' powers of two
// [rows_x], their copies per packed row [max_rows], then the partial row sums of the packed SiLU*up rows.
struct SwSums { float *xsum, *rexp, *srex, *ypart; };
static inline size_t sw_pad64(size_t n) { return (n + 63) & ~(size_t)63; }
static inline SwSums sw_sums_layout(float *sums, int rows_x, int max_rows) {
    SwSums l;
    l.xsum = sums; l.rexp = l.xsum + sw_pad64(rows_x); l.srex = l.rexp + sw_pad64(rows_x); l.ypart = l.srex + sw_pad64(max_rows);
    if (!sw_tuning().row_scale) l.rexp = l.srex = nullptr;             // every consumer takes null as "all ones"
    return l;
}
static inline size_t sw_sums_bytes(size_t T, size_t P, size_t I) { return (2 * sw_pad64(T) + sw_pad64(P) + P * (I / 8 + 1)) * 4; }

enum { SW_ST_LOGITS = 0, SW_ST_TOPK, SW_ST_DISPATCH, SW_ST_GATEUP, SW_ST_DOWN, SW_ST_SH_GATEUP, SW_ST_SH_DOWN, SW_ST_COMBINE, SW_NSTAGES };
#define SW_PROF_MAX_CALLS 512
static const char *const sw_stage_names[SW_NSTAGES] = {
    "router_logits", "route_topk", "dispatch", "q4_gateup", "q4_down", "shared_gateup", "shared_down", "combine"};

// record the event that closes stage `stage` (stage -1 = start of the call)
static inline void sw_prof_mark(SwMoeCtx *c, int stage, cudaStream_t st) {
    if (!c->prof_on || c->prof_calls >= SW_PROF_MAX_CALLS) return;
    cudaEventRecord(c->prof_ev[(size_t)c->prof_calls * (SW_NSTAGES + 1) + stage + 1], st);
}

static size_t sw_align(size_t n) { return (n + 255) & ~(size_t)255; }

extern "C" int sw_moe_ctx_create(SwMoeCtx **out, int dev, int max_tokens, int max_experts, int max_topk,
                                 int max_D, int max_I, int max_SI) {
    if (!out) return sw_fail("ctx_create: null out");
    *out = nullptr;
    if (max_tokens <= 0 || max_experts <= 0 || max_experts > SW_MAX_EXPERTS || max_topk <= 0 ||
        max_topk > SW_MAX_TOPK || max_D <= 0 || max_I <= 0 || max_SI < 0)
        return sw_fail("ctx_create: bad limits (experts <= %d, topk <= %d)", SW_MAX_EXPERTS, SW_MAX_TOPK);
    if (dev < 0 || dev >= SW_MAX_DEVICES) return sw_fail("ctx_create: device %d outside [0,%d)", dev, SW_MAX_DEVICES);
    sw_tuning();                                   // the SW_* variables are read here, once, not on the call path
    SW_CUDA(cudaSetDevice(dev));
    SwMoeCtx *c = new SwMoeCtx();
    c->dev = dev; c->maxT = max_tokens; c->maxE = max_experts; c->maxK = max_topk;
    c->maxD = max_D; c->maxI = max_I; c->maxSI = max_SI;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { const cudaError_t e = cudaGetLastError(); sw_moe_ctx_destroy(c); return sw_cuda_fail(e, "cudaGetDeviceProperties"); }
    c->num_sms = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->aux, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->cpy, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_res, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_pack, cudaEventDisableTiming) != cudaSuccess) {
        const cudaError_t e = cudaGetLastError();
        sw_moe_ctx_destroy(c);                     // releases whatever was created before the failure
        return sw_cuda_fail(e, "cudaStreamCreate");
    }

    const size_t T = max_tokens, E = max_experts, K = max_topk, D = max_D, I = max_I, SI = max_SI, P = T * K;
    size_t sizes[] = {
        T * (E + 1) * 4,      // scores (one more column for the shared expert's logit of the shared-pool policy)
        P * 4, P * 4,         // sel, w
        256,                  // G
        E * 4, E * 4, E * 4,  // gexp gbeg gcnt
        P * 4, P * 4,         // grow rowof
        256,                  // status
        sw_dispatch_scratch_ints(P, E) * 4,   // scratch of the many-CTA dispatch
        P * I * 4,            // glu
        P * D * 4,            // slots
        T * 4 + 256,          // row_gate: per-token weight of a gated shared expert
        T * (SI ? SI : 1) * 4,// sglu
        (((D + 255) / 256) * T * 2 * (SI ? SI : 1) + ((SI + 255) / 256 + 1) * T * D) * 4,   // so: slice partials of the shared expert
        T * D * 4,            // routed
        T * D * 4, T * D * 4, // dx, dout
        T * D * 4,            // xp
        sw_sums_bytes(T, P, I),  // sums
        T * D * 4,            // spk
        P * D * 4,            // um.xg: gathered fp16 hi + lo token rows
        (P / 32 + E + 64) * 8 + 256,    // um.chunks + nchunks (chunks of 32 rows at least)
        ((size_t)((D + 127) / 128) * (T < 128 ? T : 128) + ((size_t)c->num_sms * 32 * 256 + E - 1) / E + T + 64) * (E + 1) * 8   // rpart
    };
    size_t total = 0; for (size_t s : sizes) total += sw_align(s);
    if (sw_malloc(&c->block, total) != cudaSuccess) {
        cudaGetLastError(); c->block = nullptr; sw_moe_ctx_destroy(c);
        return sw_fail("ctx_create: cudaMalloc of %zu bytes failed", total);
    }
    char *p = (char *)c->block; int i = 0;
    auto take = [&](void) { void *q = p; p += sw_align(sizes[i++]); return q; };
    c->r.scores = (float *)take(); c->r.sel = (int *)take(); c->r.w = (float *)take(); c->r.G = (int *)take();
    c->r.gexp = (int *)take(); c->r.gbeg = (int *)take(); c->r.gcnt = (int *)take();
    c->r.grow = (int *)take(); c->r.rowof = (int *)take(); c->r.status = (int *)take();
    c->r.dpar = (int *)take(); c->r.dpar_ints = sw_dispatch_scratch_ints(P, E);
    c->glu = (float *)take(); c->slots = (float *)take(); c->row_gate = (float *)take(); c->sglu = (float *)take(); c->so = (float *)take();
    c->routed = (float *)take(); c->dx = (float *)take(); c->dout = (float *)take(); c->xp = take(); c->sums = (float *)take(); c->spk = take(); c->um.xg = take(); { char *q = (char *)take(); c->um.nchunks = (int *)q; c->um.chunks = q + 256; } c->rpart = (double *)take();
    cudaMemsetAsync(c->r.G, 0, 256, c->stream); cudaMemsetAsync(c->r.status, 0, 256, c->stream);
    cudaMemsetAsync(c->r.dpar, 0, 128, c->stream);              // the ticket of the many-CTA dispatch
    if (sw_malloc_host((void **)&c->hx, T * D * 4) != cudaSuccess || sw_malloc_host((void **)&c->hout, T * D * 4) != cudaSuccess) {
        cudaGetLastError(); sw_moe_ctx_destroy(c);
        return sw_fail("ctx_create: pinned staging allocation failed");
    }
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) { const cudaError_t e = cudaGetLastError(); sw_moe_ctx_destroy(c); return sw_cuda_fail(e, "cudaStreamSynchronize"); }
    *out = c;
    return 0;
}

extern "C" void sw_moe_ctx_destroy(SwMoeCtx *c) {
    if (!c) return;
    cudaSetDevice(c->dev);
    if (c->stream) { cudaStreamSynchronize(c->stream); cudaStreamDestroy(c->stream); }
    if (c->aux) { cudaStreamSynchronize(c->aux); cudaStreamDestroy(c->aux); }
    if (c->cpy) { cudaStreamSynchronize(c->cpy); cudaStreamDestroy(c->cpy); }
    if (c->ev_res) cudaEventDestroy(c->ev_res);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->ev_join) cudaEventDestroy(c->ev_join);
    if (c->ev_pack) cudaEventDestroy(c->ev_pack);
    if (c->block) cudaFree(c->block);
    if (c->hx) cudaFreeHost(c->hx);
    if (c->hout) cudaFreeHost(c->hout);
    if (c->prof_ev) {
        for (size_t i = 0; i < (size_t)SW_PROF_MAX_CALLS * (SW_NSTAGES + 1); i++) cudaEventDestroy(c->prof_ev[i]);
        free(c->prof_ev);
    }
    delete c;
}

// Argument checks that need no context and no device: descriptor ranges, layer pointers present and 16-byte
// aligned (the kernels read them with 128-bit loads and lay TMA tensor maps over the blobs).
static int sw_validate(const SwMoeDesc *d, const SwMoeLayer *L) {
    if (!d || !L) return sw_fail("null argument");
    if (d->n_experts <= 0 || d->n_experts > SW_MAX_EXPERTS) return sw_fail("n_experts=%d outside (0,%d]", d->n_experts, SW_MAX_EXPERTS);
    if (d->topk <= 0 || d->topk > SW_MAX_TOPK || d->topk > d->n_experts) return sw_fail("topk=%d invalid", d->topk);
    if (d->route_act < 0 || d->route_act > 2) return sw_fail("route_act=%d unknown", d->route_act);
    if (d->shared_mode != SW_SHARED_NONE && d->shared_mode != SW_SHARED_UNSCALED && d->shared_mode != SW_SHARED_GATED &&
        d->shared_mode != SW_SHARED_SIGMOID_GATED)
        return sw_fail("shared_mode=%d is not wired (NONE, UNSCALED, GATED and SIGMOID_GATED are)", d->shared_mode);
    if (d->shared_mode == SW_SHARED_GATED && (d->route_act != SW_ROUTE_SIGMOID || L->logit_bias || d->n_experts + 1 > SW_MAX_EXPERTS))
        return sw_fail("shared_mode GATED needs the sigmoid gate, no logit bias and at most %d experts", SW_MAX_EXPERTS - 1);
    if (d->shared_mode == SW_SHARED_SIGMOID_GATED && (!L->sh_gate_w || ((uintptr_t)L->sh_gate_w & 15)))
        return sw_fail("shared_mode SIGMOID_GATED needs sh_gate_w (f32 [D], 16-byte aligned)");
    if (L->D <= 0 || L->D % 32) return sw_fail("D=%d must be a positive multiple of 32", L->D);
    if (L->I <= 0 || L->I % 32) return sw_fail("I=%d must be a positive multiple of 32", L->I);
    if (d->shared_mode != SW_SHARED_NONE) {
        if (L->SI <= 0 || L->SI % 8) return sw_fail("SI=%d must be a positive multiple of 8", L->SI);
        if (!L->sh_gate || !L->sh_up || !L->sh_down) return sw_fail("shared expert weights missing");
    }
    if (L->gs < 0 || (L->gs > 0 && L->gs % 32)) return sw_fail("gs=%d must be 0 or a multiple of 32", L->gs);
    if (!L->router_w || !L->gu_q || !L->gu_s || !L->dn_q || !L->dn_s) return sw_fail("layer weights missing");
    if (L->router_dtype != SW_DTYPE_F32 && L->router_dtype != SW_DTYPE_BF16) return sw_fail("router_dtype=%d unknown", L->router_dtype);
    const uintptr_t al = (uintptr_t)L->router_w | (uintptr_t)L->gu_q | (uintptr_t)L->dn_q | (uintptr_t)L->gu_s | (uintptr_t)L->dn_s | (uintptr_t)L->sh_gate | (uintptr_t)L->sh_up |
                         (uintptr_t)L->sh_down;
    if (al & 15) return sw_fail("layer pointers must be 16-byte aligned (router_w, gu_q, gu_s, dn_q, dn_s, sh_*)");
    if (((uintptr_t)L->corr_bias | (uintptr_t)L->logit_bias) & 3) return sw_fail("corr_bias / logit_bias must be 4-byte aligned");
    return 0;
}
// row buffers: present and 16-byte aligned (float4 / uint4 accesses)
static int sw_validate_rows(const void *a, const void *b, const void *c3, const char *what) {
    if (!a || !b || !c3) return sw_fail("%s: null buffer", what);
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c3) & 15) return sw_fail("%s: row buffers must be 16-byte aligned", what);
    return 0;
}
extern "C" int sw_moe_validate(const SwMoeDesc *d, const SwMoeLayer *L, const void *x, const void *out) {
    if (sw_validate(d, L)) return -1;
    return sw_validate_rows(x, out, x, "validate");
}

static int sw_check(const SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, int T) {
    if (!c) return sw_fail("null argument");
    if (sw_validate(d, L)) return -1;
    if (T < 0 || T > c->maxT) return sw_fail("T=%d outside [0,%d]", T, c->maxT);
    if (d->n_experts > c->maxE) return sw_fail("n_experts=%d outside (0,%d]", d->n_experts, c->maxE);
    if (d->topk > c->maxK) return sw_fail("topk=%d invalid", d->topk);
    if (L->D > c->maxD) return sw_fail("D=%d must be a multiple of 32 and <= %d", L->D, c->maxD);
    if (L->I > c->maxI) return sw_fail("I=%d must be a multiple of 32 and <= %d", L->I, c->maxI);
    if (d->shared_mode != SW_SHARED_NONE && L->SI > c->maxSI) return sw_fail("SI=%d must be a multiple of 8 and <= %d", L->SI, c->maxSI);
    // the context's device becomes current (a host may drive several GPUs from one thread)
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != c->dev) {
        cudaGetLastError();
        if (cudaSetDevice(c->dev) != cudaSuccess) return sw_cuda_fail(cudaGetLastError(), "cudaSetDevice");
    }
    return 0;
}

static void sw_resident(const SwMoeDesc *d, const SwMoeLayer *L, int *lo, int *cnt) {
    if (L->expert_cnt > 0) { *lo = L->expert_lo; *cnt = L->expert_cnt; }
    else { *lo = 0; *cnt = d->n_experts; }
}

// gate/up then down for the groups in `a` (a.q/a.s/a.X/a.Y/KD/OUT are filled here).
// x: f32 rows; xp: scratch for the packed copy of x (rows_x rows); glu: scratch
// [max_rows, I] (f32 or packed, same size); slots: [max_rows, D] f32.
// Expert path: 2 = TMA-staged tensor-core kernels (default when the driver exports the
// tensor-map encoder), 1 = cp.async tensor-core kernels, 0 = CUDA-core f32 kernels.
// SW_EXPERT_PATH=tma|mma|simt|umma overrides.
// 3 = tcgen05/TMEM grouped GEMM, chosen when groups average SW_UMMA_MIN_ROWS (8) rows or more.
static int sw_expert_path(int D, int I, int rows, int groups) {
    const SwTuning &t = sw_tuning();
    const int pref = t.expert_pref;
    if (pref == 0 || D % 128 || I % 128) return 0;
    if (pref == 1 || !sw_tma_available()) return 1;
    if (pref == 4) return 2;
    if (pref == 3 || (groups > 0 && rows >= (long long)t.umma_min_rows * groups)) return 3;
    return 2;
}

// Which expert kernels a call will use: 0 CUDA cores, 1 mma.sync + cp.async, 2 mma.sync + TMA, 3 tcgen05.
// forced >= 0 (SW_OPT_EXPERT_PATH) asks for that family; it is still lowered when the shapes do not fit it.
// Every family reads the blobs 16 bytes at a time: alignment is checked at the entry points, not here.
static int sw_resolve_path(const SwQ4Args &a, int D, int I, const SwUmmaScratch *um, int forced = -1) {
    int path = a.gs > 0 ? 0 : sw_expert_path(D, I, a.max_rows, a.max_groups);   // group scales: CUDA-core kernels
    // Between 8 and 16 rows per group the tcgen05 kernels win only by what they save on a whole layer's weights (measured
    // with every expert resident); a shard of the experts does a fraction of that work under the same three extra
    // launches, so an expert-parallel rank stays on the streaming kernels there, as it was measured.
    if (path == 3 && forced < 0 && sw_tuning().expert_pref == 2 && a.expert_cnt < a.max_groups &&
        (long long)a.max_rows < 16LL * a.max_groups) path = 2;
    if (forced >= 0 && a.gs == 0) {
        path = forced;
        if (path > 0 && (D % 128 || I % 128)) path = 0;
        if (path >= 2 && !sw_tma_available()) path = 1;
    }
    if (path == 3 && (!um || I % 128 || D % 256)) path = 2;                   // the tcgen05 kernels walk whole tile pairs
    return path;
}

// x_packed: the packed copy of x (xp), its row sums and its rows' powers of two are already in flight or done (the
// caller ordered them before this call's stream position).
static int sw_run_experts(const SwLaunchCfg &cfg, SwQ4Args a, const void *gu_q, const float *gu_s,
                          const void *dn_q, const float *dn_s, const float *x, int rows_x, void *xp,
                          float *glu, float *slots, float *sums, int *status, int D, int I,
                          void (*mark)(void *, int), void *mark_ctx, const SwUmmaScratch *um = nullptr, bool x_packed = false,
                          int *path_out = nullptr, int umma_terms = 2, int forced_path = -1, const float **row_back = nullptr) {
    const int path = sw_resolve_path(a, D, I, um, forced_path);
    if (path_out) *path_out = path;
    // *row_back: null, or per row of x the power of two whose square the caller's combine step still has to apply
    if (row_back) *row_back = nullptr;
    if (path == 3) {
        // tcgen05 path: gather + split the token rows in packed-slot order, build the chunk list, two grouped GEMMs
        const long long nexp = a.expert_cnt > 4096 ? 4096 : a.expert_cnt;
        // groups averaging at most 12 rows: chunks of 32 rows and a deeper ring of smaller slots.  Measured: the Laguna-shaped
        // layer at 256 tokens (10 rows per group) 0.658 ms this way, 0.708 with the large-group geometry, 0.695 on the
        // streaming kernels; the very large layer at 1024 tokens (16 rows per group) 4.33 ms this way, 4.05 with the large one.
        const bool small = (long long)a.max_rows <= 12LL * a.max_groups;
        const int P = a.max_rows, max_chunks = P / sw_umma_chunk_rows(small) + a.max_groups;
        __half *xh = (__half *)um->xg, *xl = xh + (size_t)P * D;
        __half *gh = (__half *)glu, *gl = gh + (size_t)P * I;
        const SwSums sl = sw_sums_layout(sums, rows_x, a.max_rows);
        if (sl.rexp && sw_launch_row_exp(cfg, x, rows_x, D, sl.rexp)) return -1;
        if (sw_launch_umma_gather(cfg, x, a.grow, a.G + 1, P, D, xh, umma_terms == 2 ? xl : nullptr, status, sl.rexp, sl.srex)) return -1;
        if (sw_launch_umma_chunks(cfg, a, um->nchunks, um->chunks, small)) return -1;
        a.q = (const uint8_t *)gu_q; a.s = gu_s; a.KD = D; a.OUT = I;
        if (sw_launch_q4_umma(cfg, a, xh, xl, gh, gl, um->nchunks, um->chunks, max_chunks, status, nexp * 2 * I, true, umma_terms, sl.srex, small)) return -1;
        if (mark) mark(mark_ctx, 0);
        a.q = (const uint8_t *)dn_q; a.s = dn_s; a.KD = I; a.OUT = D;
        if (sw_launch_q4_umma(cfg, a, gh, gl, slots, nullptr, um->nchunks, um->chunks, max_chunks, status, nexp * D, false, umma_terms, nullptr, small)) return -1;
        if (!row_back) return -1;                                      // every caller of this path has a combine step
        *row_back = sl.rexp;
        if (mark) mark(mark_ctx, 1);
        return 0;
    }
    if (path > 0) {
        const SwSums sl = sw_sums_layout(sums, rows_x, a.max_rows);
        float *xsum = sl.xsum, *ypart = sl.ypart;
        if (!x_packed && sw_launch_pack_act(cfg, x, xp, xsum, rows_x, D, sl.rexp, status)) return -1;
        const long long nexp = a.expert_cnt > 4096 ? 4096 : a.expert_cnt;   // bounds the tensor map when the caller gave no count
        a.q = (const uint8_t *)gu_q; a.s = gu_s; a.KD = D; a.OUT = I;
        int parts;
        if (path == 2) {
            int mt = (long long)a.max_groups * ((I + 63) / 64) >= (long long)cfg.num_sms * 4 ? 2 : 1;
            if (sw_tuning().tma_mt) mt = sw_tuning().tma_mt;
            SwMmaIO io{xp, xsum, 1, glu, ypart, status, sl.rexp, sl.srex};
            if (sw_launch_q4_tma(cfg, a, io, status, nexp * 2 * I, true, mt)) return -1;
            parts = sw_q4_tma_parts(I, mt);
        } else {
            const int mt = sw_q4_mma_mt(cfg, a, true);
            SwMmaIO io{xp, xsum, 1, glu, ypart, status, sl.rexp, sl.srex};
            if (sw_launch_q4_mma(cfg, a, io, true, mt)) return -1;
            parts = I / (8 * mt);
        }
        if (mark) mark(mark_ctx, 0);
        a.q = (const uint8_t *)dn_q; a.s = dn_s; a.KD = I; a.OUT = D;
        SwMmaIO io2{glu, ypart, parts, slots, nullptr, status, sl.srex, nullptr};
        if (path == 2) {
            int mt = (long long)a.max_groups * ((D + 127) / 128) >= (long long)cfg.num_sms * 4 ? 2 : 1;
            if (sw_tuning().tma_mt) mt = sw_tuning().tma_mt;
            if (sw_launch_q4_tma(cfg, a, io2, status, nexp * D, false, mt)) return -1;
        } else {
            if (sw_launch_q4_mma(cfg, a, io2, false, sw_q4_mma_mt(cfg, a, false))) return -1;
        }
        if (mark) mark(mark_ctx, 1);
        return 0;
    }
    a.q = (const uint8_t *)gu_q; a.s = gu_s; a.X = x; a.Y = glu; a.KD = D; a.OUT = I;
    if (sw_launch_q4_gateup(cfg, a)) return -1;
    if (mark) mark(mark_ctx, 0);
    a.q = (const uint8_t *)dn_q; a.s = dn_s; a.X = glu; a.Y = slots; a.KD = I; a.OUT = D;
    if (sw_launch_q4_down(cfg, a)) return -1;
    if (mark) mark(mark_ctx, 1);
    return 0;
}

// router logits + gate + top-k; fp64 tensor-core logits when D is a multiple of 32
static int sw_logits_topk(SwMoeCtx *c, const SwLaunchCfg &cfg, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T,
                          bool mark) {
    const int E = d->n_experts, K = d->topk;
    // few pairs: the last CTA of the top-k kernel groups them (one launch less on the critical path);
    // many pairs: the 1024-thread dispatch kernel
    const bool fuse = (long long)T * K <= 4096;
    const SwRouting *dr = fuse ? &c->r : nullptr;
    unsigned *ticket = fuse ? (unsigned *)(c->r.status + 16) : nullptr;
    const int force_simt = sw_tuning().force_simt;
    // shared-pool policy: the router's last row is the shared expert's logit; its normalised weight lands in row_gate
    const int ns = d->shared_mode == SW_SHARED_GATED ? 1 : 0;
    const float pool_scale = d->route_scale * (L->route_global_scale != 0.f ? L->route_global_scale : 1.f);
    float *rg = ns ? c->row_gate : nullptr;
    if (!force_simt && L->D % 32 == 0) {
        const int KS = sw_router_slices(c->num_sms, T, L->D, E + ns);
        if (sw_launch_router_dmma(cfg, x, L->router_w, L->router_dtype, c->rpart, T, L->D, E + ns, KS)) return sw_fail("router launch failed");
        if (mark) sw_prof_mark(c, SW_ST_LOGITS, cfg.stream);
        if (sw_launch_route_topk(cfg, c->r.scores, c->rpart, KS, L->logit_bias, L->corr_bias, d->use_corr_bias, d->route_act,
                                 d->norm_topk, T, E, K, c->r.sel, c->r.w, dr, ticket, ns, pool_scale, rg)) return sw_fail("route_topk launch failed");
    } else {
        if (sw_launch_router_logits(cfg, x, L->router_w, L->router_dtype, L->logit_bias, c->r.scores, T, L->D, E + ns)) return sw_fail("router_logits launch failed");
        if (mark) sw_prof_mark(c, SW_ST_LOGITS, cfg.stream);
        if (sw_launch_route_topk(cfg, c->r.scores, nullptr, 0, nullptr, L->corr_bias, d->use_corr_bias, d->route_act,
                                 d->norm_topk, T, E, K, c->r.sel, c->r.w, dr, ticket, ns, pool_scale, rg)) return sw_fail("route_topk launch failed");
    }
    if (mark) sw_prof_mark(c, SW_ST_TOPK, cfg.stream);
    if (!fuse && sw_launch_dispatch(cfg, c->r, T, K, E)) return sw_fail("dispatch launch failed");
    return 0;
}

static int sw_route_impl(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T, cudaStream_t st) {
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    const int E = d->n_experts, K = d->topk;
    if (sw_logits_topk(c, cfg, d, L, x, T, false)) return -1;      // the top-k kernel's last CTA also runs the dispatch
    c->last_stream = st; c->lastT = T; c->lastK = K; c->lastE = E; c->lastES = E + (d->shared_mode == SW_SHARED_GATED ? 1 : 0);
    return 0;
}

static int sw_expert_stage(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T, cudaStream_t st) {
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    int lo, cnt; sw_resident(d, L, &lo, &cnt);
    const int K = d->topk, E = d->n_experts;
    SwQ4Args a{};
    a.gexp = c->r.gexp; a.gbeg = c->r.gbeg; a.gcnt = c->r.gcnt; a.G = c->r.G; a.grow = c->r.grow;
    a.expert_lo = lo; a.expert_cnt = cnt;
    a.max_rows = T * K; a.max_groups = E < T * K ? E : T * K; a.gs = L->gs;
    if (sw_run_experts(cfg, a, L->gu_q, L->gu_s, L->dn_q, L->dn_s, x, T, c->xp, c->glu, c->slots, c->sums, c->r.status, L->D, L->I, nullptr, nullptr, &c->um, false, &c->last_path, c->umma_terms, c->forced_path, &c->row_back))
        return sw_fail("expert launch failed");
    return 0;
}

// Shared expert: so[T,D] = down(silu(gate x) * (up x)).  Tensor-core path when the
// widths are multiples of 32; `pk` is scratch for the packed copy of x, sglu holds
// the packed (or f32) intermediate.
static int sw_shared_run(const SwLaunchCfg &cfg, const SwMoeLayer *L, const float *x, int T, void *pk, float *sglu, float *spart,
                         float **so, int *so_slices, void (*mark)(void *, int), void *mark_ctx, int *status = nullptr) {
    const int force_simt = sw_tuning().force_simt;
    if (!force_simt && T >= 128 && L->D % 64 == 0 && L->SI % 64 == 0 && sw_umma_available() && status) {
        // many rows: dense tcgen05 GEMMs; pk holds the planar bf16 hi|lo copy of x, sglu the planar hi|lo SiLU*up rows
        __nv_bfloat16 *xh = (__nv_bfloat16 *)pk, *xl = xh + (size_t)T * L->D;
        __nv_bfloat16 *gh = (__nv_bfloat16 *)sglu, *gl = gh + (size_t)T * L->SI;
        if (sw_launch_pack_bf16_planar(cfg, x, xh, xl, T, L->D)) return -1;
        if (sw_launch_bf16_umma(cfg, L->sh_gate, L->sh_up, xh, xl, gh, gl, T, L->D, L->SI, status, true)) return -1;
        if (mark) mark(mark_ctx, 0);
        if (sw_launch_bf16_umma(cfg, L->sh_down, nullptr, gh, gl, spart, nullptr, T, L->SI, L->D, status, false)) return -1;
        if (mark) mark(mark_ctx, 1);
        *so = spart; *so_slices = 1;
        return 0;
    }
    if (!force_simt && L->D % 32 == 0 && L->SI % 32 == 0) {
        const int ks1 = sw_shared_slices(cfg.num_sms, (L->SI + 7) / 8, L->D);
        const int ks2 = sw_shared_slices(cfg.num_sms, (L->D + 15) / 16, L->SI);
        if (sw_launch_pack_bf16(cfg, x, pk, T, L->D)) return -1;
        if (sw_launch_bf16_mma(cfg, L->sh_gate, L->sh_up, pk, spart, T, L->D, L->SI, ks1, true)) return -1;
        if (sw_launch_shared_glu(cfg, spart, ks1, T, L->SI, sglu)) return -1;
        if (mark) mark(mark_ctx, 0);
        float *dpart = spart + (size_t)ks1 * T * 2 * L->SI;
        if (sw_launch_bf16_mma(cfg, L->sh_down, nullptr, sglu, dpart, T, L->SI, L->D, ks2, false)) return -1;
        if (mark) mark(mark_ctx, 1);
        *so = dpart; *so_slices = ks2;
        return 0;
    }
    float *o = spart;
    if (sw_launch_bf16_gateup(cfg, x, L->sh_gate, L->sh_up, sglu, T, L->D, L->SI)) return -1;
    if (mark) mark(mark_ctx, 0);
    if (sw_launch_bf16_rows(cfg, sglu, L->sh_down, o, T, L->SI, L->D)) return -1;
    if (mark) mark(mark_ctx, 1);
    *so = o; *so_slices = 1;
    return 0;
}

static int sw_shared_stage(SwMoeCtx *c, const SwMoeLayer *L, const float *x, int T, cudaStream_t st, float **so, int *so_slices) {
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    if (sw_shared_run(cfg, L, x, T, c->spk, c->sglu, c->so, so, so_slices, nullptr, nullptr, c->r.status)) return sw_fail("shared expert launch failed");
    return 0;
}
// the per-token weight of the shared expert: none (plain add), the pool weight the router left in row_gate, or the
// one-row sigmoid gate computed here
static int sw_shared_gate(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T, cudaStream_t st, const float **gate) {
    *gate = nullptr;
    if (d->shared_mode == SW_SHARED_GATED) *gate = c->row_gate;
    if (d->shared_mode == SW_SHARED_SIGMOID_GATED) {
        SwLaunchCfg cfg{c->num_sms, st, c->dev};
        if (sw_launch_row_gate(cfg, x, L->sh_gate_w, c->row_gate, T, L->D)) return sw_fail("shared gate launch failed");
        *gate = c->row_gate;
    }
    return 0;
}

extern "C" int sw_moe_route(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T, void *stream) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (sw_validate_rows(x, x, x, "route")) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    return sw_route_impl(c, d, L, x, T, st);
}

extern "C" int sw_moe_experts(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, float *routed, int T, void *stream) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (sw_validate_rows(x, routed, x, "experts")) return -1;
    if (c->lastT != T || c->lastK != d->topk || c->lastE != d->n_experts) return sw_fail("experts: no matching sw_moe_route before this call");
    cudaStream_t st = (cudaStream_t)stream;
    if (sw_expert_stage(c, d, L, x, T, st)) return -1;
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    int lo, cnt; sw_resident(d, L, &lo, &cnt);
    if (sw_launch_combine(cfg, c->slots, c->r.rowof, c->r.sel, c->r.w, nullptr, 0, routed, T, d->topk, L->D, 1.f, 0, lo, cnt, nullptr, c->row_back)) return sw_fail("combine launch failed");
    return 0;
}

SwRouting *sw_ctx_routing(SwMoeCtx *c) { return &c->r; }
void sw_ctx_info(const SwMoeCtx *c, int *dev, int *num_sms, int *maxT, void **aux_stream) {
    if (dev) *dev = c->dev;
    if (num_sms) *num_sms = c->num_sms;
    if (maxT) *maxT = c->maxT;
    if (aux_stream) *aux_stream = (void *)c->aux;
}

// routed[T,D] = sum over the resident experts of w * expert(x) for routing GIVEN by the caller: sel [T,K] int32 (rank
// order; SW_NO_EXPERT = -1 entries contribute nothing) and w [T,K] f32 in device memory.  The rows are grouped by
// expert on the device exactly as after sw_moe_route.  For drivers that route elsewhere (another GPU, the host).
extern "C" int sw_moe_experts_routed(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x,
                                     const int *sel, const float *w, float *routed, int T, void *stream) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (sw_validate_rows(x, routed, x, "experts_routed")) return -1;
    if (!sel || !w) return sw_fail("experts_routed: null routing");
    cudaStream_t st = (cudaStream_t)stream;
    const int K = d->topk, E = d->n_experts;
    const size_t nb = (size_t)T * K * 4;
    if (sel != c->r.sel) SW_CUDA(cudaMemcpyAsync(c->r.sel, sel, nb, cudaMemcpyDeviceToDevice, st));
    if (w != c->r.w) SW_CUDA(cudaMemcpyAsync(c->r.w, w, nb, cudaMemcpyDeviceToDevice, st));
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    if (sw_launch_dispatch(cfg, c->r, T, K, E)) return sw_fail("dispatch launch failed");
    c->last_stream = st; c->lastT = T; c->lastK = K; c->lastE = E; c->lastES = E;
    if (sw_expert_stage(c, d, L, x, T, st)) return -1;
    int lo, cnt; sw_resident(d, L, &lo, &cnt);
    if (sw_launch_combine(cfg, c->slots, c->r.rowof, c->r.sel, c->r.w, nullptr, 0, routed, T, K, L->D, 1.f, 0, lo, cnt, nullptr, c->row_back)) return sw_fail("combine launch failed");
    return 0;
}

extern "C" int sw_moe_shared(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, int T, void *stream) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    c->shared_T = -1;
    if (T == 0 || d->shared_mode == SW_SHARED_NONE) return 0;
    if (sw_validate_rows(x, x, x, "shared")) return -1;
    float *so = nullptr; int so_slices = 1;
    if (sw_shared_stage(c, L, x, T, (cudaStream_t)stream, &so, &so_slices)) return -1;
    if (d->shared_mode == SW_SHARED_SIGMOID_GATED) { const float *gt; if (sw_shared_gate(c, d, L, x, T, (cudaStream_t)stream, &gt)) return -1; }
    c->shared_T = T; c->shared_so = so; c->shared_slices = so_slices;
    return 0;
}

extern "C" int sw_moe_finish(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, const float *routed, float *out, int T, void *stream) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (sw_validate_rows(x, routed, out, "finish")) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    const int has_shared = d->shared_mode != SW_SHARED_NONE;
    float *so = nullptr; int so_slices = 1;
    const float *gate = nullptr;
    if (has_shared && c->shared_T == T) {                                     // left by sw_moe_shared (with its gate)
        so = c->shared_so; so_slices = c->shared_slices; c->shared_T = -1;
        if (d->shared_mode == SW_SHARED_GATED || d->shared_mode == SW_SHARED_SIGMOID_GATED) gate = c->row_gate;
    } else if (has_shared) {
        if (sw_shared_stage(c, L, x, T, st, &so, &so_slices) || sw_shared_gate(c, d, L, x, T, st, &gate)) return -1;
    }
    // shared-pool policy: the weights already carry route_scale
    const float scale = d->shared_mode == SW_SHARED_GATED ? 1.f : d->route_scale;
    if (sw_launch_finish(cfg, routed, so, so_slices, out, T, L->D, scale, has_shared, gate)) return sw_fail("finish launch failed");
    return 0;
}

// accumulate: out += MoE(x) (the reference's residual add); else out = MoE(x)
static int sw_forward_impl(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, float *out, int T, void *stream, bool accumulate);

extern "C" int sw_moe_forward(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, float *out, int T, void *stream) {
    SW_GATE();
    return sw_forward_impl(c, d, L, x, out, T, stream, true);
}

// h += MoE(rmsnorm(h) * norm_w): the reference's layer tail (c/laguna.c:1119,1126) with the residual stream h kept
// on the device; the normalised rows live in the context until the block has consumed them.
extern "C" int sw_moe_forward_norm(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, float *h, const float *norm_w, float eps, int T, void *stream) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (sw_validate_rows(h, norm_w, h, "forward_norm")) return -1;
    SwLaunchCfg cfg{c->num_sms, (cudaStream_t)stream, c->dev};
    if (sw_launch_rmsnorm(cfg, h, norm_w, c->dx, T, L->D, eps)) return sw_fail("rmsnorm launch failed");
    return sw_forward_impl(c, d, L, c->dx, h, T, stream, true);
}
// y[T,D] = rmsnorm(x) * w on the device (c/moe_math.h:58-62); x == y is allowed.
extern "C" int sw_rmsnorm(const float *x, const float *w, float *y, int T, int D, float eps, void *stream) {
    if (!x || !w || !y || T < 0 || D <= 0 || (D & 3)) return sw_fail("rmsnorm: bad argument (D must be a multiple of 4)");
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return sw_fail("rmsnorm: buffers must be 16-byte aligned");
    if (T == 0) return 0;
    int dev = 0, sms = 0;
    SW_CUDA(cudaGetDevice(&dev));
    SW_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    SwLaunchCfg cfg{sms, (cudaStream_t)stream, dev};
    if (sw_launch_rmsnorm(cfg, x, w, y, T, D, eps)) return sw_fail("rmsnorm launch failed");
    return 0;
}

static int sw_forward_impl(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, float *out, int T, void *stream, bool accumulate) {
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (sw_validate_rows(x, out, x, "forward")) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    SwLaunchCfg cfg{c->num_sms, st, c->dev};
    const int E = d->n_experts, K = d->topk;
    int lo, cnt; sw_resident(d, L, &lo, &cnt);
    const int has_shared = d->shared_mode != SW_SHARED_NONE;

    struct MarkCtx { SwMoeCtx *c; cudaStream_t st; } mc{c, st};
    auto smark = [](void *p, int which) { MarkCtx *m = (MarkCtx *)p; sw_prof_mark(m->c, which == 0 ? SW_ST_SH_GATEUP : SW_ST_SH_DOWN, m->st); };
    float *so = nullptr; int so_slices = 1;
    const float *gate = nullptr;                   // per-token weight of a gated shared expert
    // The shared expert depends only on x: outside stage profiling it runs on the
    // context's second stream, forked here and joined before the combine.
    const bool overlap = has_shared && !c->prof_on;
    SwQ4Args a{};
    a.gexp = c->r.gexp; a.gbeg = c->r.gbeg; a.gcnt = c->r.gcnt; a.G = c->r.G; a.grow = c->r.grow;
    a.expert_lo = lo; a.expert_cnt = cnt;
    a.max_rows = T * K; a.max_groups = E < T * K ? E : T * K; a.gs = L->gs;
    // Packing x for the mma.sync kernels depends only on x too: it goes first on the second stream, off the
    // router -> top-k -> experts chain.
    const int path = sw_resolve_path(a, L->D, L->I, &c->um, c->forced_path);
    const bool prepack = !c->prof_on && (path == 1 || path == 2);
    if (overlap || prepack) {
        SwLaunchCfg acfg{c->num_sms, c->aux, c->dev};
        SW_CUDA(cudaEventRecord(c->ev_fork, st));
        SW_CUDA(cudaStreamWaitEvent(c->aux, c->ev_fork, 0));
        if (prepack) {
            if (sw_launch_pack_act(acfg, x, c->xp, c->sums, T, L->D, sw_sums_layout(c->sums, T, T * d->topk).rexp, c->r.status)) return sw_fail("pack launch failed");
            SW_CUDA(cudaEventRecord(c->ev_pack, c->aux));
        }
    }
    if (overlap) {
        SwLaunchCfg acfg{c->num_sms, c->aux, c->dev};
        if (sw_shared_run(acfg, L, x, T, c->spk, c->sglu, c->so, &so, &so_slices, nullptr, nullptr, c->r.status)) return sw_fail("shared expert launch failed");
        if (d->shared_mode == SW_SHARED_SIGMOID_GATED && sw_shared_gate(c, d, L, x, T, c->aux, &gate)) return -1;
        SW_CUDA(cudaEventRecord(c->ev_join, c->aux));
    }

    sw_prof_mark(c, -1, st);
    if (sw_logits_topk(c, cfg, d, L, x, T, true)) return -1;       // the top-k kernel's last CTA also runs the dispatch
    sw_prof_mark(c, SW_ST_DISPATCH, st);
    c->last_stream = st; c->lastT = T; c->lastK = K; c->lastE = E; c->lastES = E + (d->shared_mode == SW_SHARED_GATED ? 1 : 0);

    auto mark = [](void *p, int which) { MarkCtx *m = (MarkCtx *)p; sw_prof_mark(m->c, which == 0 ? SW_ST_GATEUP : SW_ST_DOWN, m->st); };
    if (prepack) SW_CUDA(cudaStreamWaitEvent(st, c->ev_pack, 0));
    if (sw_run_experts(cfg, a, L->gu_q, L->gu_s, L->dn_q, L->dn_s, x, T, c->xp, c->glu, c->slots, c->sums, c->r.status, L->D, L->I, mark, &mc, &c->um, prepack, &c->last_path, c->umma_terms, c->forced_path, &c->row_back))
        return sw_fail("expert launch failed");
    if (overlap) {
        SW_CUDA(cudaStreamWaitEvent(st, c->ev_join, 0));
        sw_prof_mark(c, SW_ST_SH_GATEUP, st); sw_prof_mark(c, SW_ST_SH_DOWN, st);
    } else if (has_shared) {
        if (sw_shared_run(cfg, L, x, T, c->spk, c->sglu, c->so, &so, &so_slices, smark, &mc, c->r.status)) return sw_fail("shared expert launch failed");
        if (d->shared_mode == SW_SHARED_SIGMOID_GATED && sw_shared_gate(c, d, L, x, T, st, &gate)) return -1;
    } else {
        sw_prof_mark(c, SW_ST_SH_GATEUP, st); sw_prof_mark(c, SW_ST_SH_DOWN, st);
    }
    if (c->wait_res) SW_CUDA(cudaStreamWaitEvent(st, c->ev_res, 0));         // forward_host: the residual rows are on their way
    if (d->shared_mode == SW_SHARED_GATED) gate = c->row_gate;              // written by the top-k kernel of this call
    const int scale_bit = d->shared_mode == SW_SHARED_GATED ? 0 : 1;         // pool weights already carry route_scale
    if (sw_launch_combine(cfg, c->slots, c->r.rowof, c->r.sel, c->r.w, so, so_slices, out, T, K, L->D,
                          d->route_scale, scale_bit | (has_shared ? 2 : 0) | (accumulate ? 4 : 0), lo, cnt, gate, c->row_back)) return sw_fail("combine launch failed");
    sw_prof_mark(c, SW_ST_COMBINE, st);
    if (c->prof_on && c->prof_calls < SW_PROF_MAX_CALLS) c->prof_calls++;
    return 0;
}

// Is p page-locked host memory the device can copy from directly?
static bool sw_host_pinned(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return at.type == cudaMemoryTypeHost;
}

extern "C" int sw_moe_forward_host(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x_host, float *out_host, int T) {
    SW_GATE();
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return 0;
    if (!x_host || !out_host) return sw_fail("forward_host: null buffer");
    const size_t n = (size_t)T * L->D * sizeof(float);
    const bool xpin = sw_host_pinned(x_host), opin = sw_host_pinned(out_host);
    // x goes up straight from the caller's buffer when that is page-locked.
    const float *src = x_host;
    if (!xpin) { memcpy(c->hx, x_host, n); src = c->hx; }
    SW_CUDA(cudaMemcpyAsync(c->dx, src, n, cudaMemcpyHostToDevice, c->stream));
    if (opin && n >= 128 * 1024) {                  // (a few rows are cheaper to add on the host than to order a third stream)
        // Page-locked residual rows: they go up on a copy stream while the kernels run, the block adds into them
        // on the device, and the result comes down into the caller's buffer: no host pass over the rows at all.
        SW_CUDA(cudaMemcpyAsync(c->dout, out_host, n, cudaMemcpyHostToDevice, c->cpy));
        SW_CUDA(cudaEventRecord(c->ev_res, c->cpy));
        c->wait_res = true;
        const int rc = sw_forward_impl(c, d, L, c->dx, c->dout, T, c->stream, true);
        c->wait_res = false;
        if (rc) { cudaStreamSynchronize(c->cpy); return -1; }
        SW_CUDA(cudaMemcpyAsync(out_host, c->dout, n, cudaMemcpyDeviceToHost, c->stream));
        SW_CUDA(cudaStreamSynchronize(c->stream));
        return 0;
    }
    // Pageable residual rows: MoE(x) comes back and is added on the host; the residual never crosses the bus.
    if (sw_forward_impl(c, d, L, c->dx, c->dout, T, c->stream, false)) return -1;
    SW_CUDA(cudaMemcpyAsync(c->hout, c->dout, n, cudaMemcpyDeviceToHost, c->stream));
    SW_CUDA(cudaStreamSynchronize(c->stream));
    const float *add = c->hout;
    const size_t cnt = (size_t)T * L->D;
    for (size_t i = 0; i < cnt; i++) out_host[i] += add[i];
    return 0;
}

// ---------------------------------------------------------------------------
// CUDA-graph replay of one block call: the launches of sw_moe_forward for fixed
// (desc, layer, x, out, T) are captured once and replayed with one graph launch.
// ---------------------------------------------------------------------------
struct SwMoeGraph { cudaGraph_t graph; cudaGraphExec_t exec; SwMoeCtx *ctx; int T, K, E; int kernels; };

extern "C" int sw_moe_graph_create(SwMoeCtx *c, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, float *out, int T,
                                   SwMoeGraph **gout) {
    if (!gout) return sw_fail("graph_create: null out");
    *gout = nullptr;
    if (sw_check(c, d, L, T)) return -1;
    if (T == 0) return sw_fail("graph_create: empty batch");
    const int prof = c->prof_on; c->prof_on = 0;
    // one eager call first: function attributes, occupancy queries and tensor maps are set up outside capture
    if (sw_moe_forward(c, d, L, x, out, T, c->stream)) { c->prof_on = prof; return -1; }
    SW_CUDA(cudaStreamSynchronize(c->stream));
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { c->prof_on = prof; return sw_cuda_fail(cudaGetLastError(), "cudaStreamBeginCapture"); }
    const long long l0 = g_launches.load();
    const int rc = sw_moe_forward(c, d, L, x, out, T, c->stream);
    const int kernels = (int)(g_launches.load() - l0);
    g_launches.store(l0);                                   // captured, not launched
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    c->prof_on = prof;
    if (rc || e != cudaSuccess || !graph) { cudaGetLastError(); if (graph) cudaGraphDestroy(graph); return rc ? -1 : sw_fail("graph capture failed: %s", cudaGetErrorString(e)); }
    cudaGraphExec_t exec = nullptr;
    if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) { cudaGetLastError(); cudaGraphDestroy(graph); return sw_fail("cudaGraphInstantiate failed"); }
    SwMoeGraph *g = new SwMoeGraph{graph, exec, c, T, d->topk, d->n_experts, kernels};
    *gout = g;
    return 0;
}

// Capture of any sequence of stage calls (route / experts / shared / finish): between capture_begin and
// capture_end the caller passes sw_moe_capture_stream(ctx) as the stream of those calls; they are recorded, not
// run.  Every call in the sequence must have run once before (set-up work cannot be captured).
extern "C" void *sw_moe_capture_stream(SwMoeCtx *c) { return c ? (void *)c->stream : nullptr; }

extern "C" int sw_moe_capture_begin(SwMoeCtx *c) {
    if (!c) return sw_fail("null ctx");
    if (c->cap_on) return sw_fail("capture_begin: a capture is already open");
    SW_CUDA(cudaStreamSynchronize(c->stream));
    if (cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return sw_cuda_fail(cudaGetLastError(), "cudaStreamBeginCapture");
    c->cap_on = 1; c->cap_prof = c->prof_on; c->prof_on = 0; c->cap_l0 = g_launches.load();
    return 0;
}

extern "C" int sw_moe_capture_end(SwMoeCtx *c, SwMoeGraph **gout) {
    if (!c || !gout) return sw_fail("capture_end: null argument");
    *gout = nullptr;
    if (!c->cap_on) return sw_fail("capture_end: no capture open");
    const int kernels = (int)(g_launches.load() - c->cap_l0);
    g_launches.store(c->cap_l0);                            // captured, not launched
    c->cap_on = 0; c->prof_on = c->cap_prof;
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    if (e != cudaSuccess || !graph) { cudaGetLastError(); if (graph) cudaGraphDestroy(graph); return sw_fail("graph capture failed: %s", cudaGetErrorString(e)); }
    cudaGraphExec_t exec = nullptr;
    if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) { cudaGetLastError(); cudaGraphDestroy(graph); return sw_fail("cudaGraphInstantiate failed"); }
    *gout = new SwMoeGraph{graph, exec, c, c->lastT, c->lastK, c->lastE, kernels};
    return 0;
}

extern "C" int sw_moe_graph_launch(SwMoeGraph *g, void *stream) {
    if (!g) return sw_fail("graph_launch: null graph");
    SW_GATE();
    SW_CUDA(cudaGraphLaunch(g->exec, (cudaStream_t)stream));
    g->ctx->last_stream = (cudaStream_t)stream; g->ctx->lastT = g->T; g->ctx->lastK = g->K; g->ctx->lastE = g->E;
    sw_count_launch(g->kernels);
    return 0;
}

extern "C" void sw_moe_graph_destroy(SwMoeGraph *g) {
    if (!g) return;
    cudaGraphExecDestroy(g->exec); cudaGraphDestroy(g->graph);
    delete g;
}

extern "C" int sw_moe_get_routing(SwMoeCtx *c, int *sel, float *w, float *scores, int *G,
                                  int *gexp, int *gbeg, int *gcnt, int *grow, int *rowof) {
    if (!c) return sw_fail("null ctx");
    if (c->lastT <= 0) return sw_fail("get_routing: nothing routed yet");
    SW_CUDA(cudaStreamSynchronize(c->last_stream));
    const size_t P = (size_t)c->lastT * c->lastK, E = c->lastE;
    if (sel)    SW_CUDA(cudaMemcpy(sel, c->r.sel, P * 4, cudaMemcpyDeviceToHost));
    if (w)      SW_CUDA(cudaMemcpy(w, c->r.w, P * 4, cudaMemcpyDeviceToHost));
    if (scores) SW_CUDA(cudaMemcpy2D(scores, E * 4, c->r.scores, (size_t)(c->lastES > 0 ? c->lastES : (int)E) * 4, E * 4, (size_t)c->lastT, cudaMemcpyDeviceToHost));
    if (G)      SW_CUDA(cudaMemcpy(G, c->r.G, 4, cudaMemcpyDeviceToHost));
    if (gexp)   SW_CUDA(cudaMemcpy(gexp, c->r.gexp, E * 4, cudaMemcpyDeviceToHost));
    if (gbeg)   SW_CUDA(cudaMemcpy(gbeg, c->r.gbeg, E * 4, cudaMemcpyDeviceToHost));
    if (gcnt)   SW_CUDA(cudaMemcpy(gcnt, c->r.gcnt, E * 4, cudaMemcpyDeviceToHost));
    if (grow)   SW_CUDA(cudaMemcpy(grow, c->r.grow, P * 4, cudaMemcpyDeviceToHost));
    if (rowof)  SW_CUDA(cudaMemcpy(rowof, c->r.rowof, P * 4, cudaMemcpyDeviceToHost));
    return 0;
}

extern "C" int sw_moe_status(SwMoeCtx *c) {
    if (!c) return -1;
    int s = 0;
    if (c->last_stream) cudaStreamSynchronize(c->last_stream);
    if (cudaMemcpy(&s, c->r.status, 4, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (s && cudaMemset(c->r.status, 0, 4) != cudaSuccess) { cudaGetLastError(); return -1; }     // read and clear, like cudaGetLastError
    return s;
}

// Expert kernels of the last sw_moe_experts / sw_moe_forward call of this context:
// 0 CUDA cores (k_q4_group), 1 mma.sync + cp.async (k_q4_mma), 2 mma.sync + TMA (k_q4_tma), 3 tcgen05 + TMEM (k_q4_umma); -1 before the first call.
extern "C" int sw_moe_last_path(SwMoeCtx *c) { return c ? c->last_path : -1; }

extern "C" int sw_moe_set_option(SwMoeCtx *c, int option, int value) {
    if (!c) return sw_fail("null ctx");
    if (option == SW_OPT_UMMA_TERMS) {
        if (value != 1 && value != 2) return sw_fail("set_option: SW_OPT_UMMA_TERMS takes 1 or 2");
        c->umma_terms = value;
        return 0;
    }
    if (option == SW_OPT_EXPERT_PATH) {
        if (value < -1 || value > 3) return sw_fail("set_option: SW_OPT_EXPERT_PATH takes -1 (choose) or 0..3");
        c->forced_path = value;
        return 0;
    }
    return sw_fail("set_option: unknown option %d", option);
}

// Runs a one-CTA kernel whose bounded wait cannot succeed (limit = `iters` polls of a barrier nobody arrives at),
// clears the status word first, and returns the status bits afterwards: SW_ST_TIMEOUT (4) when the give-up path
// worked.  The context stays usable.
extern "C" int sw_moe_test_wait_timeout(SwMoeCtx *c, int iters) {
    if (!c || iters <= 0 || iters > (1 << 20)) return sw_fail("test_wait_timeout: bad argument");
    SwLaunchCfg cfg{c->num_sms, c->stream, c->dev};
    SW_CUDA(cudaMemsetAsync(c->r.status, 0, 4, c->stream));
    if (sw_launch_wait_runs_out(cfg, c->r.status, (unsigned)iters)) return sw_fail("test kernel launch failed");
    int st = 0;
    SW_CUDA(cudaMemcpyAsync(&st, c->r.status, 4, cudaMemcpyDeviceToHost, c->stream));
    SW_CUDA(cudaStreamSynchronize(c->stream));
    SW_CUDA(cudaMemsetAsync(c->r.status, 0, 4, c->stream));
    SW_CUDA(cudaStreamSynchronize(c->stream));
    return st;
}

// Host-only self-test of the per-device set-up slots and of the tensor-map cache keying (no device needed).
int sw_selftest_map_cache();
extern "C" int sw_selftest_host(void) {
    SwPerDevice slots{};
    int runs = 0;
    auto init7 = [&] { runs++; return 7; };
    if (slots.get(0, init7) != 7 || slots.get(0, init7) != 7 || runs != 1) return 101;       // device 0: set up once
    if (slots.get(1, [&] { runs++; return 9; }) != 9 || runs != 2) return 102;              // device 1 does its own set-up
    if (slots.get(0, init7) != 7 || runs != 2) return 103;
    if (slots.get(2, [&] { runs++; return -1; }) > 0 || slots.get(2, [&] { runs++; return 3; }) != 3 || runs != 4) return 104;   // a failure is not cached
    if (slots.get(SW_MAX_DEVICES, init7) > 0 || slots.get(-1, init7) > 0) return 105;
    return sw_selftest_map_cache();
}

extern "C" int sw_moe_profile(SwMoeCtx *c, int enable) {
    if (!c) return sw_fail("null ctx");
    if (enable && !c->prof_ev) {
        size_t n = (size_t)SW_PROF_MAX_CALLS * (SW_NSTAGES + 1);
        c->prof_ev = (cudaEvent_t *)malloc(n * sizeof(cudaEvent_t));
        if (!c->prof_ev) return sw_fail("profile: out of host memory");
        for (size_t i = 0; i < n; i++) SW_CUDA(cudaEventCreate(&c->prof_ev[i]));
    }
    c->prof_on = enable ? 1 : 0; c->prof_calls = 0;
    return 0;
}
extern "C" int sw_moe_profile_read(SwMoeCtx *c, float *ms, int *calls) {
    if (!c || !ms) return sw_fail("null argument");
    for (int s = 0; s < SW_NSTAGES; s++) ms[s] = 0.f;
    if (calls) *calls = c->prof_calls;
    if (!c->prof_ev || c->prof_calls == 0) return 0;
    SW_CUDA(cudaStreamSynchronize(c->last_stream));
    for (int i = 0; i < c->prof_calls; i++)
        for (int s = 0; s < SW_NSTAGES; s++) {
            float t = 0.f;
            cudaEvent_t *e = c->prof_ev + (size_t)i * (SW_NSTAGES + 1);
            SW_CUDA(cudaEventElapsedTime(&t, e[s], e[s + 1]));
            ms[s] += t;
        }
    return 0;
}
extern "C" int sw_moe_stage_count(void) { return SW_NSTAGES; }
extern "C" const char *sw_moe_stage_name(int i) { return i >= 0 && i < SW_NSTAGES ? sw_stage_names[i] : ""; }

// ===========================================================================
// lag_cuda_* drop-in tier: host pointers in, host pointers out, one sync per call.
// ===========================================================================
#define SW_LAG_TC_MIN_ROWS 16
static struct {
    int ok = 0, dev = 0, num_sms = 0;
    cudaStream_t st = nullptr;
    SwBuf dx, dy, dxp, dglu, dslot, dsums, didx, dmisc;
    SwBuf hx{nullptr, 0, true}, hy{nullptr, 0, true}, hidx{nullptr, 0, true};
} g_lag;

extern "C" int lag_cuda_init(int dev) {
    if (dev < 0 || dev >= SW_MAX_DEVICES) return -1;
    sw_tuning();
    cudaSetDeviceFlags(cudaDeviceScheduleSpin);   // many short blocking calls per token (c/backend_cuda_laguna.cu:17-21)
    cudaGetLastError();
    if (cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); return -1; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (!g_lag.st && cudaStreamCreate(&g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
    void *probe = nullptr;
    if (cudaMalloc(&probe, 1 << 20) != cudaSuccess) { cudaGetLastError(); return -1; }
    cudaFree(probe);
    g_lag.dev = dev; g_lag.num_sms = prop.multiProcessorCount; g_lag.ok = 1;
    return 0;
}
extern "C" size_t lag_cuda_free_bytes(void) {
    size_t fr = 0, to = 0;
    if (cudaMemGetInfo(&fr, &to) != cudaSuccess) { cudaGetLastError(); return 0; }
    return fr;
}
extern "C" size_t lag_cuda_total_bytes(void) {
    size_t fr = 0, to = 0;
    if (cudaMemGetInfo(&fr, &to) != cudaSuccess) { cudaGetLastError(); return 0; }
    return to;
}
extern "C" void *lag_cuda_upload(const void *h, size_t n) {
    void *d = nullptr;
    if (sw_malloc(&d, n ? n : 1) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (n && cudaMemcpy(d, h, n, cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); cudaFree(d); return nullptr; }
    return d;
}
extern "C" void lag_cuda_free(void *d) { if (d) cudaFree(d); }

// stage x (xn bytes) to the device, run `body`, bring yn bytes of dy back to y
template <typename F>
static int lag_roundtrip(float *y, const float *x, size_t xn, size_t yn, F body) {
    if (g_lag.dx.ensure(xn) || g_lag.dy.ensure(yn) || g_lag.hx.ensure(xn) || g_lag.hy.ensure(yn)) return -1;
    memcpy(g_lag.hx.p, x, xn);
    if (cudaMemcpyAsync(g_lag.dx.p, g_lag.hx.p, xn, cudaMemcpyHostToDevice, g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (body()) return -1;
    if (cudaMemcpyAsync(g_lag.hy.p, g_lag.dy.p, yn, cudaMemcpyDeviceToHost, g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (cudaStreamSynchronize(g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
    memcpy(y, g_lag.hy.p, yn);
    return 0;
}

extern "C" int lag_cuda_matmul_bf16(float *y, const float *x, const void *W, int S, int I, int O) {
    if (sw_fault_injected()) return -1;
    if (!g_lag.ok || S <= 0 || I <= 0 || O <= 0 || (I & 7)) return -1;
    if (!y || !x || !W || ((uintptr_t)W & 15)) return -1;                     // weight rows are read 16 bytes at a time
    SwLaunchCfg cfg{g_lag.num_sms, g_lag.st, g_lag.dev};
    // Batched calls (prefill, S >= 16) go to the tensor cores when the shapes fit: x as two bf16 terms (hi + lo), weights
    // exact, f32 accumulate; from 128 rows the dense tcgen05 GEMM, below mma.sync over slices of the contraction with
    // the partial sums added in slice order.  Decode-size calls keep the f32 kernels: the reference's acceptance bar for
    // this call is an ELEMENT-wise relative error (c/laguna.c:1579), which only an f32 dot meets on near-zero outputs.
    const bool tc = !sw_tuning().force_simt && S >= SW_LAG_TC_MIN_ROWS && I % 32 == 0 && O % 4 == 0;
    if (tc && S >= 128 && I % 64 == 0 && sw_umma_available()) {
        if (g_lag.dxp.ensure((size_t)S * I * 4) || g_lag.dmisc.ensure(1024)) return -1;
        return lag_roundtrip(y, x, (size_t)S * I * 4, (size_t)S * O * 4, [&] {
            __nv_bfloat16 *xh = (__nv_bfloat16 *)g_lag.dxp.p, *xl = xh + (size_t)S * I;
            int *status = (int *)g_lag.dmisc.p + 128;
            if (cudaMemsetAsync(status, 0, 4, g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
            if (sw_launch_pack_bf16_planar(cfg, (const float *)g_lag.dx.p, xh, xl, S, I)) return -1;
            return sw_launch_bf16_umma(cfg, W, nullptr, xh, xl, g_lag.dy.p, nullptr, S, I, O, status, false);
        });
    }
    if (tc) {
        const int ks = sw_shared_slices(cfg.num_sms, (O + 15) / 16, I);
        if (g_lag.dxp.ensure((size_t)S * I * 4) || g_lag.dslot.ensure((size_t)ks * S * O * 4)) return -1;
        return lag_roundtrip(y, x, (size_t)S * I * 4, (size_t)S * O * 4, [&] {
            if (sw_launch_pack_bf16(cfg, (const float *)g_lag.dx.p, g_lag.dxp.p, S, I)) return -1;
            if (sw_launch_bf16_mma(cfg, W, nullptr, g_lag.dxp.p, (float *)g_lag.dslot.p, S, I, O, ks, false)) return -1;
            return sw_launch_sum_slices(cfg, (const float *)g_lag.dslot.p, ks, (size_t)S * O, (float *)g_lag.dy.p);
        });
    }
    return lag_roundtrip(y, x, (size_t)S * I * 4, (size_t)S * O * 4, [&] {
        return sw_launch_bf16_rows(cfg, (const float *)g_lag.dx.p, W, (float *)g_lag.dy.p, S, I, O);
    });
}
extern "C" int lag_cuda_matmul_q8(float *y, const float *x, const void *W, int S, int I, int O) {
    if (sw_fault_injected()) return -1;
    if (!g_lag.ok || S <= 0 || I <= 0 || O <= 0) return -1;
    if (!y || !x || !W || (((uintptr_t)W + (size_t)I * O) & 3)) return -1;      // the f32 scales follow the int8 block
    SwLaunchCfg cfg{g_lag.num_sms, g_lag.st, g_lag.dev};
    const int8_t *q8 = (const int8_t *)W;
    const float *scale = (const float *)(q8 + (size_t)I * O);
    return lag_roundtrip(y, x, (size_t)S * I * 4, (size_t)S * O * 4, [&] {
        return sw_launch_q8_rows(cfg, (const float *)g_lag.dx.p, q8, scale, (float *)g_lag.dy.p, S, I, O);
    });
}

// index block on the device: [G | gexp(n) | gbeg(n) | gcnt(n) | grow(P) | rowof(P) | sel(P) | w(P)]
struct LagIdx { int *G, *gexp, *gbeg, *gcnt, *grow, *rowof, *sel; float *w; };
static int lag_stage_idx(LagIdx *d, const int *gexp, const int *gbeg, const int *gcnt, int G,
                         const int *grow, const int *rowof, const float *w, int P) {
    size_t nint = 64 + (size_t)3 * G + 3 * (size_t)P, bytes = (nint + P) * 4;
    if (g_lag.didx.ensure(bytes) || g_lag.hidx.ensure(bytes)) return -1;
    int *h = (int *)g_lag.hidx.p;
    for (int i = 0; i < 64; i++) h[i] = 0;
    h[0] = G; h[1] = P;                             // groups, packed rows
    int *hp = h + 64;
    memcpy(hp, gexp, (size_t)G * 4); hp += G;
    memcpy(hp, gbeg, (size_t)G * 4); hp += G;
    memcpy(hp, gcnt, (size_t)G * 4); hp += G;
    memcpy(hp, grow, (size_t)P * 4); hp += P;
    memcpy(hp, rowof, (size_t)P * 4); hp += P;
    for (int i = 0; i < P; i++) hp[i] = 0;          // sel: every pair resident (expert 0 of a 1-expert window)
    hp += P;
    memcpy(hp, w, (size_t)P * 4);
    if (cudaMemcpyAsync(g_lag.didx.p, h, bytes, cudaMemcpyHostToDevice, g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
    int *dp = (int *)g_lag.didx.p;
    d->G = dp; dp += 64;
    d->gexp = dp; dp += G; d->gbeg = dp; dp += G; d->gcnt = dp; dp += G;
    d->grow = dp; dp += P; d->rowof = dp; dp += P; d->sel = dp; dp += P; d->w = (float *)dp;
    return 0;
}

// Core of the grouped entry points.  Expert ids in gexp index the blobs directly.
static int lag_group_core(float *acc, const float *x, const void *gu_q, const float *gu_s,
                          const void *dn_q, const float *dn_s,
                          const int *gexp, const int *gbeg, const int *gcnt, int G,
                          const int *grow, const int *rowof, const float *w, int S, int K, int I, int D) {
    if (sw_fault_injected()) return -1;
    if (!g_lag.ok || S <= 0 || K <= 0 || G <= 0 || (D % 32) || (I % 32)) return -1;
    if (!acc || !x || !gu_q || !gu_s || !dn_q || !dn_s || !gexp || !gbeg || !gcnt || !grow || !rowof || !w) return -1;
    if (((uintptr_t)gu_q | (uintptr_t)gu_s | (uintptr_t)dn_q | (uintptr_t)dn_s) & 15) return -1;   // 128-bit loads, TMA tensor maps
    const int P = S * K;
    if (g_lag.dglu.ensure((size_t)P * I * 4) || g_lag.dslot.ensure((size_t)P * D * 4) || g_lag.dxp.ensure((size_t)S * D * 4) ||
        g_lag.dsums.ensure(sw_sums_bytes(S, P, I))) return -1;
    LagIdx ix;
    if (lag_stage_idx(&ix, gexp, gbeg, gcnt, G, grow, rowof, w, P)) return -1;
    SwLaunchCfg cfg{g_lag.num_sms, g_lag.st, g_lag.dev};
    return lag_roundtrip(acc, x, (size_t)S * D * 4, (size_t)S * D * 4, [&] {
        SwQ4Args a{};
        a.gexp = ix.gexp; a.gbeg = ix.gbeg; a.gcnt = ix.gcnt; a.G = ix.G; a.grow = ix.grow;
        a.expert_lo = 0; a.expert_cnt = 0x7fffffff; a.max_groups = G; a.max_rows = P;
        const float *row_back = nullptr;
        if (sw_run_experts(cfg, a, gu_q, gu_s, dn_q, dn_s, (const float *)g_lag.dx.p, S, g_lag.dxp.p,
                           (float *)g_lag.dglu.p, (float *)g_lag.dslot.p, (float *)g_lag.dsums.p, ix.G + 32, D, I, nullptr, nullptr,
                           nullptr, false, nullptr, 2, -1, &row_back)) return -1;
        return sw_launch_combine(cfg, (const float *)g_lag.dslot.p, ix.rowof, ix.sel, ix.w, nullptr, 0, (float *)g_lag.dy.p,
                                 S, K, D, 1.f, 0, 0, 1, nullptr, row_back);
    });
}

extern "C" int lag_cuda_moe_group(float *acc, const float *x, const void *gu_q, const float *gu_s,
                                  const void *dn_q, const float *dn_s,
                                  const int *gexp, const int *gbeg, const int *gcnt, int G,
                                  const int *grow, const int *rowof, const float *w,
                                  int S, int K, int I, int D) {
    return lag_group_core(acc, x, gu_q, gu_s, dn_q, dn_s, gexp, gbeg, gcnt, G, grow, rowof, w, S, K, I, D);
}

extern "C" int lag_cuda_moe_experts(float *out, const float *x, const void *gu_q, const float *gu_s,
                                    const void *dn_q, const float *dn_s,
                                    const int *sel, const float *w, int K, int I, int D) {
    if (K <= 0 || K > 4096) return -1;
    // one row: each selection is its own group of one packed row, kept in the caller's order
    int *tmp = (int *)malloc((size_t)K * 5 * sizeof(int));
    if (!tmp) return -1;
    int *gbeg = tmp, *gcnt = tmp + K, *grow = tmp + 2 * K, *rowof = tmp + 3 * K;
    for (int k = 0; k < K; k++) { gbeg[k] = k; gcnt[k] = 1; grow[k] = 0; rowof[k] = k; }
    int rc = lag_group_core(out, x, gu_q, gu_s, dn_q, dn_s, sel, gbeg, gcnt, K, grow, rowof, w, 1, K, I, D);
    free(tmp);
    return rc;
}

extern "C" int lag_cuda_expert_q4(float *out, const float *x, const void *p13, const void *s13,
                                  const void *p2, const void *s2, int I, int D) {
    const int zero = 0, one = 1; const float w1 = 1.f;
    return lag_group_core(out, x, p13, (const float *)s13, p2, (const float *)s2, &zero, &zero, &one, 1, &zero, &zero, &w1, 1, 1, I, D);
}

// fp4 pair (c/backend_cuda_laguna.h:83-99): same conventions as the int4 calls.
extern "C" int lag_cuda_matmul_fp4(float *y, const float *x, const void *packed, const void *es, int S, int I, int O) {
    if (sw_fault_injected()) return -1;
    if (!g_lag.ok || S <= 0 || O <= 0 || I <= 0 || (I & 31)) return -1;          // scale blocks are 32 wide
    if (!y || !x || !packed || !es || ((uintptr_t)packed & 15)) return -1;
    SwLaunchCfg cfg{g_lag.num_sms, g_lag.st, g_lag.dev};
    return lag_roundtrip(y, x, (size_t)S * I * 4, (size_t)S * O * 4, [&] {
        return sw_launch_fp4_rows(cfg, (const float *)g_lag.dx.p, packed, es, (float *)g_lag.dy.p, S, I, O);
    });
}

extern "C" int lag_cuda_moe_experts_fp4(float *out, const float *x, const void *gu_q, const void *gu_es,
                                        const void *dn_q, const void *dn_es, const int *sel, const float *w, int K,
                                        int I, int D, float limit) {
    if (sw_fault_injected()) return -1;
    if (!g_lag.ok || K < 0 || K > 4096 || I <= 0 || D <= 0 || (D & 31) || (I & 31)) return -1;
    if (K > 0 && (!sel || !w)) return -1;
    if (!out || !x || !gu_q || !gu_es || !dn_q || !dn_es || (((uintptr_t)gu_q | (uintptr_t)dn_q) & 15)) return -1;
    const size_t ib = (size_t)(K > 0 ? K : 1) * 8;                                // sel [K] int32, then w [K] f32
    if (g_lag.didx.ensure(ib) || g_lag.hidx.ensure(ib) || g_lag.dglu.ensure((size_t)(K + 1) * I * 4) ||
        g_lag.dslot.ensure((size_t)(K + 1) * D * 4)) return -1;
    if (K > 0) { memcpy(g_lag.hidx.p, sel, (size_t)K * 4); memcpy((char *)g_lag.hidx.p + (size_t)K * 4, w, (size_t)K * 4); }
    SwLaunchCfg cfg{g_lag.num_sms, g_lag.st, g_lag.dev};
    return lag_roundtrip(out, x, (size_t)D * 4, (size_t)D * 4, [&] {
        if (K > 0 && cudaMemcpyAsync(g_lag.didx.p, g_lag.hidx.p, (size_t)K * 8, cudaMemcpyHostToDevice, g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
        const int *dsel = (const int *)g_lag.didx.p;
        const float *dw = (const float *)((const char *)g_lag.didx.p + (size_t)K * 4);
        return sw_launch_fp4_experts(cfg, (const float *)g_lag.dx.p, gu_q, gu_es, dn_q, dn_es, dsel, dw, K, I, D, limit,
                                     (float *)g_lag.dglu.p, (float *)g_lag.dslot.p, (float *)g_lag.dy.p);
    });
}

extern "C" int lag_cuda_matmul_q4(float *y, const float *x, const void *packed, const void *scale, int S, int I, int O) {
    if (sw_fault_injected()) return -1;
    if (!g_lag.ok || S <= 0 || O <= 0 || I <= 0 || (I % 32)) return -1;
    if (!y || !x || !packed || !scale || (((uintptr_t)packed | (uintptr_t)scale) & 15)) return -1;
    // a single group of S packed rows through the row-output form of the grouped kernel
    if (g_lag.dmisc.ensure(256 * 4)) return -1;
    int h[256] = {0};
    h[0] = 1; h[64] = 0; h[65] = 0; h[66] = S;      // G | gexp gbeg gcnt
    if (cudaMemcpyAsync(g_lag.dmisc.p, h, sizeof h, cudaMemcpyHostToDevice, g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (cudaStreamSynchronize(g_lag.st) != cudaSuccess) { cudaGetLastError(); return -1; }   // h is a stack buffer
    int *dm = (int *)g_lag.dmisc.p;
    SwLaunchCfg cfg{g_lag.num_sms, g_lag.st, g_lag.dev};
    // batched calls (S >= 16): the rows are one group of the TMA-staged tensor-core int4 kernel (row-output form);
    // decode-size calls keep the f32 kernel (element-wise relative bar of the reference's self-test, c/laguna.c:1593)
    const bool tc = !sw_tuning().force_simt && sw_tuning().expert_pref >= 2 && S >= SW_LAG_TC_MIN_ROWS && I % 128 == 0 && sw_tma_available();
    if (tc && (g_lag.dxp.ensure((size_t)S * I * 4) || g_lag.dsums.ensure(((size_t)S + 64) * 4))) return -1;
    return lag_roundtrip(y, x, (size_t)S * I * 4, (size_t)S * O * 4, [&] {
        SwQ4Args a{};
        a.G = dm; a.gexp = dm + 64; a.gbeg = dm + 65; a.gcnt = dm + 66; a.grow = nullptr;
        a.expert_lo = 0; a.expert_cnt = 1; a.max_groups = 1; a.max_rows = S;
        a.q = (const uint8_t *)packed; a.s = (const float *)scale; a.X = (const float *)g_lag.dx.p; a.Y = (float *)g_lag.dy.p;
        a.KD = I; a.OUT = O;
        if (tc) {
            if (sw_launch_pack_act(cfg, (const float *)g_lag.dx.p, g_lag.dxp.p, (float *)g_lag.dsums.p, S, I, nullptr, nullptr)) return -1;
            SwMmaIO io{g_lag.dxp.p, (const float *)g_lag.dsums.p, 1, g_lag.dy.p, nullptr, nullptr, nullptr, nullptr};
            const int mt = (O + 127) / 128 >= cfg.num_sms * 4 ? 2 : 1;
            return sw_launch_q4_tma(cfg, a, io, dm + 128, O, false, mt);
        }
        return sw_launch_q4_down(cfg, a);
    });
}
