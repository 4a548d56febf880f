// Shared declarations of the MoE-block kernels and their host launchers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <atomic>
#include <mutex>

#define SW_FULL_MASK 0xffffffffu
#define SW_MAX_EXPERTS 1024     // top-k keeps <= 32 scores per lane
#define SW_MAX_TOPK 32
#define SW_NO_EXPERT (-1)       // sel entry of a (row, rank) pair that selects nothing: skipped by dispatch and combine

// Status bits written by kernels into SwRouting::status.
#define SW_ST_BAD_EXPERT 1
#define SW_ST_BAD_ROW    2
#define SW_ST_TIMEOUT    4     // a bounded device-side wait ran out
#define SW_ST_RANGE      8     // an activation left the fp16 range of the tensor-core paths and was clamped to +-65504

// Routing + dispatch arrays of one block call (device pointers).  Names follow
// the reference's host arrays (c/laguna.c:709-723).
struct SwRouting {
    float *scores;   // [T,E] logits in, gate scores out
    int   *sel;      // [T,K] expert ids, rank order
    float *w;        // [T,K] combine weights
    int   *G;        // [2]   number of non-empty groups; number of (row, rank) pairs that selected an expert
    int   *gexp, *gbeg, *gcnt;   // [E]
    int   *grow;     // [T*K] packed row -> token row
    int   *rowof;    // [T*K] (token, rank) -> packed row
    int   *status;   // [1]
    int   *dpar;     // scratch of the many-CTA dispatch (null: one CTA does it), dpar_ints ints
    size_t dpar_ints;
};
// ints of scratch the many-CTA dispatch needs for P pairs over E experts
size_t sw_dispatch_scratch_ints(size_t P, size_t E);

struct SwLaunchCfg {
    int num_sms;
    cudaStream_t stream;
    int dev;           // CUDA device the stream belongs to (function attributes and occupancy are kept per device)
};

// Set-up results that CUDA keeps per device (opt-in to large shared memory, resident CTAs per SM): one slot per
// device, filled once under a process-wide mutex, so a second context on another GPU does its own set-up.
#define SW_MAX_DEVICES 64
std::mutex &sw_setup_mutex();
struct SwPerDevice {
    std::atomic<int> v[SW_MAX_DEVICES];
    // The cached value of `dev` (> 0).  `init` computes it the first time and returns > 0, or <= 0 on failure,
    // which is returned uncached so that the next call tries again.
    template <typename F> int get(int dev, F init) {
        if (dev < 0 || dev >= SW_MAX_DEVICES) return -1;
        int cur = v[dev].load(std::memory_order_acquire);
        if (cur > 0) return cur;
        std::lock_guard<std::mutex> g(sw_setup_mutex());
        cur = v[dev].load(std::memory_order_relaxed);
        if (cur > 0) return cur;
        cur = init();
        if (cur > 0) v[dev].store(cur, std::memory_order_release);
        return cur;
    }
};

// Tuning knobs (SW_* environment variables), read once per process -- when the first context is created or
// lag_cuda_init runs -- never on the call path.
struct SwTuning {
    int expert_pref;     // SW_EXPERT_PATH: 2 default, 3 umma, 4 tma always, 1 mma, 0 simt
    int umma_min_rows;   // SW_UMMA_MIN_ROWS: mean rows per group from which the tcgen05 kernels are used
    int row_scale;       // SW_ROW_SCALE (default 1): 0 switches the per-token power-of-two normalisation of the tensor-core paths off (measurements)
    int force_simt;      // SW_FORCE_SIMT
    int tma_mt;          // SW_TMA_MT: 0 = choose, 1 or 2
    int tma_p;           // SW_TMA_P: ring depth of the TMA decode kernels (0 = default)
    int mma_mt;          // SW_MMA_MT
    int fail_after;      // SW_FAIL_AFTER: > 0 makes the n-th and later device allocations of this library fail (host-side failure injection)
};
const SwTuning &sw_tuning();

void sw_count_launch(int n = 1);

// internal views of a context for the other translation units (sw_ep.cu, sw_glm.cu)
struct SwMoeCtx;
SwRouting *sw_ctx_routing(SwMoeCtx *c);
void sw_ctx_info(const SwMoeCtx *c, int *dev, int *num_sms, int *maxT, void **aux_stream);
int sw_fail_text(const char *fmt, ...);          // sets the thread's last-error text, returns -1

// sw_route.cu
int sw_launch_router_logits(const SwLaunchCfg &c, const float *x, const void *W, int w_dtype,
                            const float *logit_bias, float *rl, int T, int D, int E);
int sw_router_slices(int num_sms, int T, int D, int E);
int sw_launch_router_dmma(const SwLaunchCfg &c, const float *x, const void *W, int w_dtype, double *part,
                          int T, int D, int E, int KS);
// part != NULL: logits are first formed as (float)(sum of KS fp64 partials [KS][T][E]) + lbias
int sw_launch_route_topk(const SwLaunchCfg &c, float *scores, const double *part, int KS, const float *lbias,
                         const float *corr_bias, int use_bias,
                         int route_act, int norm_topk, int T, int E, int K, int *sel, float *w,
                         const SwRouting *dr = nullptr, unsigned *ticket = nullptr,
                         int ns = 0, float pool_scale = 1.f, float *row_gate = nullptr);
// row_gate[t] = sigmoid(x[t] . g) with the dot accumulated in fp64 (a one-row gate of the shared expert)
int sw_launch_row_gate(const SwLaunchCfg &c, const float *x, const float *g, float *row_gate, int T, int D);
int sw_launch_dispatch(const SwLaunchCfg &c, const SwRouting &r, int T, int K, int E);

// sw_experts.cu
struct SwQ4Args {
    const uint8_t *q; const float *s;     // blob of the first resident expert
    const float *X; float *Y;
    const int *gexp, *gbeg, *gcnt, *G, *grow;
    int KD;            // contraction length
    int OUT;           // gate/up: I (pairs of rows); down: rows
    int expert_lo, expert_cnt;
    int max_groups;    // upper bound on *G known on the host
    int max_rows;      // upper bound on rows of all groups together (T*K)
    int gs;            // 0: one scale per row; >0: one scale per gs columns (CUDA-core kernels only)
};
int sw_launch_q4_gateup(const SwLaunchCfg &c, const SwQ4Args &a);
int sw_launch_q4_down(const SwLaunchCfg &c, const SwQ4Args &a);
// sw_mma.cu: tensor-core path (needs KD % 128 == 0)
struct SwMmaIO {
    const void *XP;        // packed activation rows
    const float *xsum;     // [rows, xsum_parts] partial sums of each packed row's values
    int xsum_parts;
    void *Y;               // gate/up: packed rows; down: f32 rows
    float *ypart;          // gate/up only: [rows, OUT/(8*mt)] sums of what each item wrote
    int *status;           // device status word (may be null): SW_ST_RANGE when a value had to be clamped to the fp16 range
    // Per-row powers of two (both may be null = 1).  gate/up: rex[token row] = 2^e the packed row was divided by; the
    // kernel also copies it to srex_out[packed row].  down: rex[packed row]; the outputs are multiplied by its square.
    const float *rex;
    float *srex_out;
};
// rexp (may be null): normalise every row by a power of two and store it there (see k_pack_act)
int sw_launch_pack_act(const SwLaunchCfg &c, const float *x, void *xp, float *rowsum, int rows, int KD, float *rexp, int *status);
int sw_q4_mma_mt(const SwLaunchCfg &c, const SwQ4Args &a, bool gateup);
int sw_launch_q4_mma(const SwLaunchCfg &c, const SwQ4Args &a, const SwMmaIO &io, bool gateup, int mt);
// sw_tma.cu: TMA-staged variant of the int4 products
bool sw_tma_available();
int sw_q4_tma_parts(int OUT, int mt);
int sw_launch_q4_tma(const SwLaunchCfg &c, const SwQ4Args &a, const SwMmaIO &io, int *status, long long rows_total, bool gateup, int mt);
int sw_launch_wait_runs_out(const SwLaunchCfg &c, int *status, unsigned limit);
// sw_umma.cu: tcgen05/TMEM grouped GEMM for groups with many rows
bool sw_umma_available();
int sw_launch_row_exp(const SwLaunchCfg &c, const float *x, int rows, int KD, float *rexp);
int sw_launch_umma_gather(const SwLaunchCfg &c, const float *x, const int *grow, const int *npairs, int P, int KD, void *hi, void *lo, int *status,
                          const float *rexp, float *srex);
int sw_umma_chunk_rows(bool small);   // rows per chunk: 128, or 32 for launches of small groups (deeper ring of smaller slots)
int sw_launch_umma_chunks(const SwLaunchCfg &c, const SwQ4Args &a, int *nchunks, void *chunks, bool small);
int sw_launch_q4_umma(const SwLaunchCfg &c, const SwQ4Args &a, const void *act_hi, const void *act_lo, void *Y0, void *Y1,
                      const int *nchunks, const void *chunks, int max_chunks, int *status, long long wrows_total, bool gateup, int terms,
                      const float *srex, bool small);
int sw_launch_pack_bf16_planar(const SwLaunchCfg &c, const float *x, void *hi, void *lo, int rows, int KD);
int sw_launch_bf16_umma(const SwLaunchCfg &c, const void *W0, const void *W1, const void *act_hi, const void *act_lo,
                        void *Y0, void *Y1, int T, int KD, int O, int *status, bool gateup);
int sw_launch_pack_bf16(const SwLaunchCfg &c, const float *x, void *xp, int rows, int KD);
int sw_shared_slices(int num_sms, int mblocks, int KD);
int sw_launch_bf16_mma(const SwLaunchCfg &c, const void *W0, const void *W1, const void *XP, float *part,
                       int T, int KD, int O, int KS, bool gateup);
int sw_launch_shared_glu(const SwLaunchCfg &c, const float *part, int KS, int T, int SI, void *out);
int sw_launch_bf16_gateup(const SwLaunchCfg &c, const float *x, const void *Wg, const void *Wu,
                          float *sglu, int T, int D, int SI);
int sw_launch_bf16_rows(const SwLaunchCfg &c, const float *x, const void *W, float *y, int T, int I, int O);
int sw_launch_q8_rows(const SwLaunchCfg &c, const float *x, const int8_t *W, const float *scale,
                      float *y, int T, int I, int O);
// out/routed combine.  mode bits: 1 = multiply by route_scale, 2 = add `add` rows
// (shared expert output), 4 = accumulate into out (else overwrite).
// `add` holds add_slices consecutive [T,D] arrays that are summed in order.
int sw_launch_combine(const SwLaunchCfg &c, const float *slots, const int *rowof, const int *sel,
                      const float *w, const float *add, int add_slices, float *out, int T, int K, int D,
                      float route_scale, int mode, int expert_lo, int expert_cnt, const float *row_gate = nullptr,
                      const float *row_back = nullptr);   // row_back[t]: power of two whose square multiplies row t's routed sum
int sw_launch_finish(const SwLaunchCfg &c, const float *routed, const float *add, int add_slices, float *out,
                     int T, int D, float route_scale, int has_add, const float *row_gate = nullptr);
int sw_launch_rmsnorm(const SwLaunchCfg &c, const float *x, const float *w, float *y, int T, int D, float eps);
int sw_launch_sum_slices(const SwLaunchCfg &c, const float *part, int KS, size_t n, float *y);
// fp4 (e2m1 + ue8m0 block-32) products of the lag_cuda_* tier (sw_fp4.cu)
int sw_launch_fp4_rows(const SwLaunchCfg &c, const float *x, const void *P, const void *ES, float *y, int S, int I, int O);
int sw_launch_fp4_experts(const SwLaunchCfg &c, const float *x, const void *gu_q, const void *gu_es, const void *dn_q,
                          const void *dn_es, const int *sel, const float *w, int K, int I, int D, float limit,
                          float *glu, float *part, float *out);

