/* sabrewing_b200.h -- C-ABI of the B200-native MoE-block backend.
 *
 * Two layers of entry points live in one shared library (libsabrewing_b200.so):
 *
 *  1. The lag_cuda_* functions.  Names, argument order, pointer domains (host vs
 *     device) and return conventions are those of the reference's Laguna CUDA tier,
 *     c/backend_cuda_laguna.h:25-75, so an engine built against that header links
 *     against this library unchanged.  0 = ok, -1 = error (the caller falls back to
 *     its CPU path), upload returns NULL on failure.  Blocking: each call returns
 *     after its stream has been synchronised.  Not thread-safe (one global stream
 *     and scratch, like the reference, c/backend_cuda_laguna.cu:11-15).
 *
 *  2. The sw_moe_* functions: a descriptor-level, device-resident MoE block.  The
 *     descriptor is the reference's MoeDesc (c/moe_arch.h:33-41); the layer struct
 *     carries what the reference's MoeHooks reach through engine state
 *     (c/moe_arch.h:45-55, c/laguna.c:572-617): router weights, correction bias,
 *     the int4 expert container and the bf16 shared expert.  One call runs
 *     route -> top-k -> group-by-expert -> int4 gate/up -> SiLU*up -> int4 down ->
 *     rank-order combine -> *route_scale -> + shared expert -> out += , with no
 *     host round trip (what c/moe_block.h:18-54 and c/laguna.c:689-787 do on the CPU).
 *
 * All sizes are element counts unless stated.  No function aborts the process.
 */
#ifndef SABREWING_B200_H
#define SABREWING_B200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------- */
/* 1. Drop-in Laguna tier (c/backend_cuda_laguna.h)                           */
/* ------------------------------------------------------------------------- */

/* c/backend_cuda_laguna.h:25 -- select device, create the stream. 0 = ok. */
int    lag_cuda_init(int dev);
/* c/backend_cuda_laguna.h:26-27 */
size_t lag_cuda_free_bytes(void);
size_t lag_cuda_total_bytes(void);
/* c/backend_cuda_laguna.h:28-29 -- copy n host bytes into new device memory. */
void  *lag_cuda_upload(const void *h, size_t n);
void   lag_cuda_free(void *d);
/* c/backend_cuda_laguna.h:32 -- y[S,O] = x[S,I] . W^T, W device bf16 [O,I], x/y host f32. */
int    lag_cuda_matmul_bf16(float *y, const float *x, const void *W, int S, int I, int O);
/* c/backend_cuda_laguna.h:36 -- W device [int8 O*I][f32 scale O]. */
int    lag_cuda_matmul_q8(float *y, const float *x, const void *W, int S, int I, int O);
/* c/backend_cuda_laguna.h:39-40 -- W device packed int4 [O,I/2] + f32 row scales [O]. */
int    lag_cuda_matmul_q4(float *y, const float *x, const void *packed,
                          const void *scale, int S, int I, int O);
/* c/backend_cuda_laguna.h:44-46 -- out[D] = W2 . siluglu(W13 . x), one expert, one row. */
int    lag_cuda_expert_q4(float *out, const float *x,
                          const void *p13, const void *s13,
                          const void *p2, const void *s2, int I, int D);
/* c/backend_cuda_laguna.h:51-54 -- out[D] = sum_k w[k]*expert(sel[k], x); sel/w host. */
int    lag_cuda_moe_experts(float *out, const float *x,
                            const void *gu_q, const float *gu_s,
                            const void *dn_q, const float *dn_s,
                            const int *sel, const float *w, int K, int I, int D);
/* c/backend_cuda_laguna.h:70-75 -- grouped experts over S rows with host index
 * arrays; acc[S,D] = unscaled weighted routed sum, summed in rank order. */
int    lag_cuda_moe_group(float *acc, const float *x,
                          const void *gu_q, const float *gu_s,
                          const void *dn_q, const float *dn_s,
                          const int *gexp, const int *gbeg, const int *gcnt, int G,
                          const int *grow, const int *rowof, const float *w,
                          int S, int K, int I, int D);
/* c/backend_cuda_laguna.h:83-84 -- fp4: W device e2m1 codes [O,I/2] (low nibble = even column), es device
 * ue8m0 exponent bytes [O,I/32]; value = lut[code] * 2^(es-127).  I % 32 == 0. */
int    lag_cuda_matmul_fp4(float *y, const float *x, const void *packed,
                           const void *es, int S, int I, int O);
/* c/backend_cuda_laguna.h:93-98 -- out[D] = sum_k w[k]*expert(sel[k], x) over a resident fp4 layer, one token,
 * SwiGLU clamped asymmetrically (gate <= limit, |up| <= limit); experts are added in the order given. */
int    lag_cuda_moe_experts_fp4(float *out, const float *x,
                                const void *gu_q, const void *gu_es,
                                const void *dn_q, const void *dn_es,
                                const int *sel, const float *w, int K,
                                int I, int D, float limit);

/* ------------------------------------------------------------------------- */
/* 2. Descriptor-level device-resident MoE block                              */
/* ------------------------------------------------------------------------- */

/* Router gate activation.  0/1 are the reference's MoeRouteAct (c/moe_arch.h:22);
 * 2 applies the reference's softplusf (c/moe_math.h:54) as the gate -- the
 * reference has no router that uses it, so it is checked against the CPU
 * restatement only. */
enum { SW_ROUTE_SIGMOID = 0, SW_ROUTE_SOFTMAX = 1, SW_ROUTE_SOFTPLUS = 2 };
/* Shared-expert policy.  0, 1 and 3 carry the values of the reference's MoeSharedMode
 * (c/moe_arch.h:25-30); NONE and UNSCALED are the two that moe_block wires
 * (c/moe_block.h:44-51).  GATED is the inkling engine's policy (c/inkling.c:1038-1043):
 * the router has one more row, the shared expert's logit; the combine weights are the
 * sigmoid scores of the K picks and of the shared expert, normalised to sum 1 over all
 * K + 1 and multiplied by route_scale * route_global_scale, so the shared expert enters the
 * sum like one more pick and nothing is scaled afterwards (sigmoid gate only, one shared
 * expert).  SIGMOID_GATED is the qwen35 engine's (c/qwen35.c:684-699): out += routed *
 * route_scale + sigmoid(x . sh_gate_w) * shared(x), a one-row gate per token.  SCALED (2)
 * is not wired in the reference and is refused here. */
enum { SW_SHARED_NONE = 0, SW_SHARED_UNSCALED = 1, SW_SHARED_GATED = 3, SW_SHARED_SIGMOID_GATED = 4 };
enum { SW_DTYPE_F32 = 0, SW_DTYPE_BF16 = 1 };

/* Same fields, order and types as MoeDesc (c/moe_arch.h:33-41). */
typedef struct {
    int   n_experts;
    int   topk;
    int   route_act;
    int   use_corr_bias;
    int   norm_topk;
    float route_scale;
    int   shared_mode;
} SwMoeDesc;

/* Device-resident weights of one layer.  The int4 container is the reference's
 * fused per-layer layout (c/laguna.c:92-96,415-419; c/moe_quant.h:13-14): expert e's
 * gate rows then up rows start at row e*2I of gu_q [E*2I, D/2] (scales gu_s [E*2I]),
 * its down rows at row e*D of dn_q [E*D, I/2] (scales dn_s [E*D]); value =
 * nibble-8, low nibble = even column.  When only a contiguous range of experts is
 * resident on this GPU (expert-parallel shard), gu_q/gu_s/dn_q/dn_s point at the
 * rows of expert expert_lo and expert_cnt says how many follow; pairs routed to
 * other experts contribute nothing here. */
typedef struct {
    int D, I, SI;              /* hidden, routed ffn width, shared ffn width (0 if none) */
    int router_dtype;          /* SW_DTYPE_F32 or SW_DTYPE_BF16 */
    const void  *router_w;     /* [E, D] */
    const float *corr_bias;    /* [E] or NULL: added to the score for SELECTION only */
    const float *logit_bias;   /* [E] or NULL: added to the logits before the gate */
    const void  *gu_q; const float *gu_s;
    const void  *dn_q; const float *dn_s;
    const void  *sh_gate, *sh_up, *sh_down;   /* bf16 [SI,D], [SI,D], [D,SI] or NULL */
    int expert_lo, expert_cnt; /* resident expert range; expert_cnt<=0 means all */
    int gs;                    /* 0: one f32 scale per weight row (c/moe_quant.h:13-14).  >0 (multiple of 32):
                                  one scale per gs columns, gu_s [E*2I, ceil(D/gs)], dn_s [E*D, ceil(I/gs)]
                                  -- the reference's group-scaled int4, c/quant.h:167-202 */
    const float *sh_gate_w;    /* SW_SHARED_SIGMOID_GATED: f32 [D], the shared expert's one-row gate; else NULL */
    float route_global_scale;  /* SW_SHARED_GATED: the layer's gate.global_scale (0 is read as 1) */
} SwMoeLayer;

typedef struct SwMoeCtx SwMoeCtx;

/* Scratch and staging for blocks of up to max_tokens rows.  Allocates device
 * memory once; sw_moe_forward itself allocates nothing. */
int  sw_moe_ctx_create(SwMoeCtx **ctx, int dev, int max_tokens, int max_experts, int max_topk,
                       int max_D, int max_I, int max_SI);
void sw_moe_ctx_destroy(SwMoeCtx *ctx);

/* out[T,D] += MoE(x[T,D]); x, out device f32; stream is a cudaStream_t passed
 * through as given (NULL = CUDA's default stream).  Asynchronous on that stream.  Residual semantics
 * follow c/moe_block.h:51 / c/laguna.c:781. */
int  sw_moe_forward(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                    const float *x, float *out, int T, void *stream);
/* The layer tail with the residual stream resident on the device: h[T,D] += MoE(rmsnorm(h) * norm_w)
 * (c/laguna.c:1119 then :1126; rmsnorm_row c/moe_math.h:58-62: sum of squares in double).  The
 * normalised rows stay in the context; nothing crosses the host.  sw_rmsnorm is the norm alone. */
int  sw_moe_forward_norm(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer, float *h,
                         const float *norm_w, float eps, int T, void *stream);
int  sw_rmsnorm(const float *x, const float *w, float *y, int T, int D, float eps, void *stream);
/* Same through HOST buffers: pinned staging, H2D, the block, D2H, stream sync --
 * the shape of a reference lag_cuda_* call (c/backend_cuda_laguna.cu:516-546).
 * out_host is read and updated in place. */
int  sw_moe_forward_host(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                         const float *x_host, float *out_host, int T);

/* CUDA-graph replay of sw_moe_forward for fixed (desc, layer, x, out, T): create
 * runs the block once eagerly (out is updated by that call too), captures a second
 * call and instantiates it; launch replays it on `stream`.  The context's scratch
 * is shared, so replays of graphs of one context must not overlap on the GPU. */
typedef struct SwMoeGraph SwMoeGraph;
int  sw_moe_graph_create(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                         const float *x, float *out, int T, SwMoeGraph **graph);
int  sw_moe_graph_launch(SwMoeGraph *graph, void *stream);
void sw_moe_graph_destroy(SwMoeGraph *graph);

/* Stages, for expert-parallel drivers and for parity checks.  route: router
 * logits -> gate -> top-k -> weights -> group-by-expert, results kept in ctx.
 * experts: routed[T,D] = sum over resident experts of w*expert (unscaled, rank
 * order, overwrites).  finish: out += routed*route_scale + shared(x). */
int  sw_moe_route(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                  const float *x, int T, void *stream);
int  sw_moe_experts(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                    const float *x, float *routed, int T, void *stream);
int  sw_moe_finish(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                   const float *x, const float *routed, float *out, int T, void *stream);
/* Optional: the shared expert of x[T,D] (c/laguna.c:596-602) ahead of time, e.g. on another stream while the
 * routed rows are exchanged between GPUs.  The result stays in ctx and is consumed by the next sw_moe_finish
 * with the same T, which then skips its own shared-expert pass; ordering the two streams is the caller's job. */
int  sw_moe_shared(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer,
                   const float *x, int T, void *stream);
/* Capture of a sequence of stage calls into a graph: begin, then the calls with sw_moe_capture_stream(ctx) as
 * their stream (recorded, not run; each must have run once before), then end.  The graph is launched and
 * destroyed like one from sw_moe_graph_create.  For drivers that interleave the stages with their own work
 * (collectives) and want one launch per segment. */
void *sw_moe_capture_stream(SwMoeCtx *ctx);
int  sw_moe_capture_begin(SwMoeCtx *ctx);
int  sw_moe_capture_end(SwMoeCtx *ctx, SwMoeGraph **graph);

/* Grouped experts for routing GIVEN by the caller: sel [T,K] int32 in rank order (-1 =
 * the pair contributes nothing) and w [T,K] f32, device memory.  routed[T,D] = sum over the
 * resident experts of w * expert(x), unscaled, overwritten; the rows are grouped by expert
 * on the device as after sw_moe_route (c/laguna.c:709-723).  For drivers that route
 * elsewhere: another GPU (sw_ep_*), or the host as the lag_cuda_* callers do. */
int  sw_moe_experts_routed(SwMoeCtx *ctx, const SwMoeDesc *desc, const SwMoeLayer *layer, const float *x,
                           const int *sel, const float *w, float *routed, int T, void *stream);

/* ------------------------------------------------------------------------- */
/* 3. Expert-parallel step over the GPUs of one node (one process per GPU)    */
/* ------------------------------------------------------------------------- */
/* Experts sharded contiguously over the ranks (rank g owns experts [g*E/N, (g+1)*E/N),
 * the first E % N ranks one more), router and shared expert replicated, T rows per
 * rank.  The reference has no multi-process layer (its multi-device code is peer
 * copies and per-device grouping on the host, c/backend_cuda.cu:1444-1466,
 * c/colibri.c:3506-3607).  One call is one step: the NCCL collectives are enqueued
 * from inside the library on the caller's stream, between its kernels.  NCCL is
 * loaded at run time (libnccl.so.2); hosts that never call sw_ep_* need none.
 *   SW_EP_REPLICATE: all-gather rows, route all N*T rows on every rank, resident
 *     experts, reduce-scatter the partial sums (decode-size batches).
 *   SW_EP_ALLTOALL: route own rows, send each row once to every GPU holding one of
 *     its experts (with ids and weights), experts there, one pre-weighted partial
 *     sum per row back, added in GPU order (large batches).  One host sync per step
 *     to size the sends.
 * sw_ep_unique_id: 128 bytes from rank 0 that every rank passes to sw_ep_create (the
 * host distributes them; any transport).  ctx must hold N*T rows.  Not thread-safe per
 * SwEp; 0 = ok, -1 = error with sw_last_error(). */
enum { SW_EP_REPLICATE = 0, SW_EP_ALLTOALL = 1 };
typedef struct SwEp SwEp;
int  sw_ep_unique_id(void *id128);
int  sw_ep_create(SwEp **ep, SwMoeCtx *ctx, const void *id128, int world, int rank, int rows_per_rank, int D, int topk);
void sw_ep_destroy(SwEp *ep);
int  sw_ep_forward(SwEp *ep, const SwMoeDesc *desc, const SwMoeLayer *layer, const float *x, float *out, int T,
                   int scheme, int timed, void *stream);
int  sw_ep_segments(SwEp *ep, float *ms, int scheme);

/* Container loader: one MoE layer of a Laguna int4 snapshot from its safetensors file(s) (a file
 * or a directory of them) straight into device memory, in the reference's container layout
 * (docs/laguna.md:34-42; names as c/laguna.c:410-446 reads them through c/st.h): router
 * `mlp.gate.weight` F32 or BF16, `mlp.experts.e_score_correction_bias`, fused packed int4
 * `mlp.experts.gate_up_proj` / `down_proj` with `.qs` row scales, bf16 `mlp.shared_expert.*`.
 * expert_cnt > 0 reads only the rows of experts [expert_lo, expert_lo + expert_cnt) (an
 * expert-parallel shard).  *layer then points at device memory owned by *handle. */
typedef struct SwLoadedLayer SwLoadedLayer;
int  sw_layer_load(const char *path, int layer_index, int dev, int expert_lo, int expert_cnt,
                   SwMoeLayer *layer, int *n_experts, SwLoadedLayer **handle);
void sw_layer_free(SwLoadedLayer *handle);

/* Routing without any allocation (no counterpart in the reference, which sizes its
 * scratch with cudaMalloc on demand, c/backend_cuda_laguna.cu:471-493): router
 * logits -> gate -> top-k -> combine weights for T <= 8 rows, n_experts <= 512,
 * D <= 8192 (D % 32 == 0).  x [T,D] f32, sel [T*K] int32 and w [T*K] f32 are device
 * buffers owned by the caller; the working memory is a fixed ~2.1 MB array inside
 * the library image that every GPU loading the library keeps until exit.  Meant
 * for hosts that cannot allocate when they need a routing decision (all free
 * device memory already given away, or no tolerance for the device-wide
 * synchronisation of an allocation).  Same ids as sw_moe_route; weights equal to
 * within one unit in the last place.  Sizes beyond the limits, NULL or misaligned
 * buffers (x, router_w: 16 bytes) return -1 with an error text.  The array is
 * shared by all calls on a GPU: calls that overlap on the device race, so order
 * them.  The first call on each device looks up the array's device address; issue
 * it outside any stream capture and at start-up: CUDA loads the module that holds
 * the array lazily, so the memory is reserved by that first call, not when the
 * library loads, and a host that has already given all device memory away by then
 * gets -1. */
int  sw_moe_route_static(const SwMoeDesc *desc, const SwMoeLayer *layer, const float *x, int T,
                         int *sel, float *w, void *stream);

/* Copy the routing of the last sw_moe_route/forward to host arrays (any may be
 * NULL): sel,w [T*K]; scores [T*E]; *G; gexp,gbeg,gcnt [E]; grow,rowof [T*K] -- the
 * arrays of c/laguna.c:709-723.  Synchronises the stream used last. */
int  sw_moe_get_routing(SwMoeCtx *ctx, int *sel, float *w, float *scores, int *G,
                        int *gexp, int *gbeg, int *gcnt, int *grow, int *rowof);

/* Device-side status word: the bits raised by the launches since the previous call of this
 * function, which clears them (0 = clean; synchronises the stream used last); bit 0: an expert id
 * outside [0,E) reached the dispatch, bit 1: a row index outside [0,T), bit 2: a
 * bounded device-side wait ran out (the kernel gave up and returned), bit 3: an
 * activation, or a SiLU(gate)*up value entering the down product, left the fp16
 * range of the tensor-core expert kernels (every path but the CUDA-core one) and was
 * clamped to +-65504: the result is then not the reference's (the reference is f32
 * throughout, c/moe_quant.h:45-217).  The kernels divide every token row by a power
 * of two on its way in and multiply back in f32 (the bar holds for inputs 1e-6 ...
 * 1e6 times the usual size, tests/test_moe_gpu.py), so in practice the bit means an
 * infinity or a NaN in the input. */
int  sw_moe_status(SwMoeCtx *ctx);
/* Context options.  SW_OPT_UMMA_TERMS: how the tcgen05 grouped GEMM (groups averaging >= 8
 * rows: prefill, large batches) feeds f32 activations to the fp16 tensor cores.
 * 1 (default) = fp16(x) alone: each activation, and each SiLU*up value entering the down
 * product, is rounded to 11 significant bits; measured relative L2 of the block output
 * against the reference's exact f32 path: 2.7e-4 on the 4096-token Laguna-shaped prefill,
 * 5.6e-5 on the 1024-token very large layer (bar 1e-3).  2 = two fp16 terms, x = hi + lo,
 * two MMAs per step: f32-level accuracy (1.2e-5 / 1.8e-5 on the same cases) at twice the
 * tensor work.  Routing is identical either way.  The decode kernels (small groups) always
 * use both terms.
 * SW_OPT_EXPERT_PATH: -1 (default) lets the library choose the expert kernels by shape
 * and mean group size; 0..3 asks for one family (numbering of sw_moe_last_path), lowered
 * when the shapes do not fit it.  For tests and measurements.
 * 0 = ok, -1 = unknown option or value. */
enum { SW_OPT_UMMA_TERMS = 1, SW_OPT_EXPERT_PATH = 2 };
int  sw_moe_set_option(SwMoeCtx *ctx, int option, int value);
/* Which expert kernels the last sw_moe_experts / sw_moe_forward of this context
 * used: 0 CUDA cores, 1 mma.sync + cp.async, 2 mma.sync + TMA, 3 tcgen05 + TMEM;
 * -1 before the first call.  For tests and benchmarks that must know the path. */
int  sw_moe_last_path(SwMoeCtx *ctx);
/* Argument checks of the block calls without a context or a device: descriptor
 * ranges, layer pointers present and 16-byte aligned, x / out present and 16-byte
 * aligned.  0 = acceptable, -1 = refused with an error text. */
int  sw_moe_validate(const SwMoeDesc *desc, const SwMoeLayer *layer, const void *x, const void *out);
/* Failure handling hooks; failures are injected on the host, never on the device.
 * sw_test_fail_after(n): the reference's COLI_GPU_FAIL_AFTER (c/backend_cuda.cu:684-692,
 * tested in c/tests/test_backend_cuda.cu:93-98): every compute entry point (the block,
 * its stages, graph launches, the lag_cuda_* products) reports failure once n calls have
 * succeeded; n = 0: every call fails; n < 0: off.  SW_FAIL_AFTER=n in the environment
 * does the same from the start.  Uploads, queries and context creation are not gated.
 * sw_test_fail_alloc(n): the n-th and every later device / page-locked allocation of this
 * library fails without calling CUDA (n <= 0: off).
 * sw_moe_test_wait_timeout: launches one CTA whose bounded barrier wait cannot succeed
 * and returns the status bits it left (bit 2 expected); the context stays usable.
 * sw_selftest_host: host-only checks of the per-device set-up slots and the tensor-map
 * cache keying, 0 = pass. */
void sw_test_fail_after(int n);
void sw_test_fail_alloc(int n);
int  sw_moe_test_wait_timeout(SwMoeCtx *ctx, int iters);
int  sw_selftest_host(void);
/* Per-stage device timing with CUDA events recorded on the call's stream between
 * the kernels of sw_moe_forward (what the reference's COLI_CUDA_PROFILE split does,
 * c/backend_cuda.cu:822-929).  enable=1 starts a fresh accumulation (up to 512
 * calls), read returns total ms per stage and the number of calls recorded. */
int  sw_moe_profile(SwMoeCtx *ctx, int enable);
int  sw_moe_profile_read(SwMoeCtx *ctx, float *ms_per_stage, int *calls);
int  sw_moe_stage_count(void);
const char *sw_moe_stage_name(int i);
/* Number of kernels launched by this library since load. */
long long sw_launch_count(void);
/* Text of the last error on the calling thread's most recent failing call. */
const char *sw_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
