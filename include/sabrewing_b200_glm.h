/* sabrewing_b200_glm.h -- the GLM engine's CUDA boundary for the MoE path, served by
 * libsabrewing_b200.so.
 *
 * Names, argument order, pointer domains and return conventions are those of the
 * reference's c/backend_cuda.h (1 = ok, 0 = failure: the engine falls back to its CPU
 * path; handles are opaque; devices are CUDA ordinals), so colibri.c built against
 * that header links against this library for the calls below.  What is here is the
 * MoE hot path and what it stands on: device set-up, resident-tensor handles, the
 * plain product, the fused expert pipelines (host rows, issue/take, device-resident)
 * and the device router with route-level top-p, plus the residual-stream primitives
 * either side of the block (RMSNorm, adds, device GEMM).  The attention and RoPE entry
 * points of c/backend_cuda.h:96-141,158-160,164-181 are not part of this path and are
 * not exported.  fmt follows the engine's QT: 0 f32, 1 int8 + row scales, 2 int4 + row
 * scales, 4 int4 + one scale per gs inputs (c/quant.h:167-202); 3 (int2) reports 0.
 */
#ifndef SABREWING_B200_GLM_H
#define SABREWING_B200_GLM_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define COLI_CUDA_MAX_DEVICES 16

/* c/backend_cuda.h:24-25 -- opaque, persistent device copy of one resident quantised tensor */
typedef struct ColiCudaTensor ColiCudaTensor;

/* c/backend_cuda.h:27-37 */
int    coli_cuda_init(const int *devices, int count);
void   coli_cuda_shutdown(void);
int    coli_cuda_device_count(void);
int    coli_cuda_device_at(int index);
int    coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes);
void   coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes);
void   coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows,
                             double *h2d_ms, double *kernel_ms, double *d2h_ms);

/* c/backend_cuda.h:39-45 -- upload without executing (capacity failures at start-up) */
int    coli_cuda_tensor_upload_g(ColiCudaTensor **tensor, const void *weights, const float *scales,
                                 int fmt, int I, int O, int device, int gs);
int    coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights, const float *scales,
                               int fmt, int I, int O, int device);
/* c/backend_cuda.h:47-58 -- y[S,O] = x[S,I] . W[O,I]^T, host x / y; first call uploads W */
int    coli_cuda_matmul(ColiCudaTensor **tensor, float *y, const float *x, const void *weights,
                        const float *scales, int fmt, int S, int I, int O, int device, int gs);
/* c/backend_cuda.h:60-64 -- y = down(silu(gate(x)) * up(x)), three resident tensors, host rows */
int    coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down,
                            float *y, const float *x, int S);
/* c/backend_cuda.h:74-92 -- packed group of same-shaped experts: x and y hold sum(rows)
 * consecutive [D] rows in call order; issue/take is the asynchronous split for <= 8 rows */
int    coli_cuda_expert_group_issue(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                    ColiCudaTensor *const *downs, const int *rows, int count, const float *x);
const float *coli_cuda_expert_group_take(int device);
int    coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                              ColiCudaTensor *const *downs, const int *rows, int count,
                              float *y, const float *x);
/* c/backend_cuda.h:128-135 */
void   coli_cuda_tensor_free(ColiCudaTensor *tensor);
size_t coli_cuda_tensor_bytes(const ColiCudaTensor *tensor);
int    coli_cuda_tensor_device(const ColiCudaTensor *tensor);
int    coli_cuda_tensor_update(ColiCudaTensor *tensor, const void *weights, const float *scales);

/* c/backend_cuda.h:137-157,161-162,182 -- resident-pipeline primitives, device pointers */
float *coli_cuda_pipe_scratch(int device, int slot, size_t bytes);
void  *coli_cuda_pipe_alloc(int device, size_t bytes);
void   coli_cuda_pipe_free(int device, void *p);
int    coli_cuda_pipe_upload(int device, void *dst, const void *src, size_t bytes);
int    coli_cuda_pipe_download(int device, const void *src, void *dst, size_t bytes);
int    coli_cuda_pipe_rmsnorm(int device, float *y_dev, const float *x_dev, const float *w_dev, int S, int D, float eps);
int    coli_cuda_pipe_rmsnorm_s(int device, float *y_dev, const float *x_dev, const float *w_dev, int S, int D,
                                float eps, int xstride, int ystride);
int    coli_cuda_pipe_silu_mul(int device, float *gate_dev, const float *up_dev, size_t n);
int    coli_cuda_pipe_add(int device, float *x_dev, const float *t_dev, size_t n);
int    coli_cuda_pipe_rows_add(int device, float *x_dev, const float *partial_dev, const int *rows_dev, int nrows, int D);
int    coli_cuda_pipe_gemm(ColiCudaTensor *t, float *y_dev, const float *x_dev, int S);
int    coli_cuda_pipe_copy2d(int device, float *dst, int dpitch, const float *src, int spitch, int width, int height);
int    coli_cuda_pipe_peer_copy(int dst_dev, float *dst, int src_dev, const float *src, size_t bytes);
int    coli_cuda_pipe_sync(int device);
/* c/backend_cuda.h:143-149 -- decode-time expert group with no host bytes: the row is pulled
 * from the home device, outputs are weighted and summed in the order given, the partial sum
 * is pushed into a slot on the home device; take adds the slots in issue order */
int    coli_cuda_expert_group_resident_issue(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                             ColiCudaTensor *const *downs, const float *weights, int count,
                                             int home_device, const float *x_src_dev, float *partial_slot_dev);
int    coli_cuda_expert_group_resident_take(int home_device, const int *devices, int n_issued,
                                            float *slots_dev, float *acc_dev, int D);
/* c/backend_cuda.h:150-153 -- router for one decode row on the device: sigmoid scores,
 * top-K of score + bias, top-p truncation (c/backend_cuda.cu:1338-1347), renormalisation,
 * routed scale; idx/w/keff on the host.  Here: D % 8 == 0, E <= 1024, Ksel <= 32, else 0. */
int    coli_cuda_pipe_router(int device, const float *x_dev, const void *rw_dev, const void *rb_dev,
                             int D, int E, int Ksel, float topp, int norm_topk, float routed_scale,
                             int *idx_host, float *w_host, int *keff_host);

#ifdef __cplusplus
}
#endif
#endif
