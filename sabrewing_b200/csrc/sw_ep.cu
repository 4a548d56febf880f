// Expert-parallel step over the GPUs of one node, as ONE host call: the exchanges are NCCL collectives
// enqueued from here on the caller's stream, between this library's kernels.
//
// Experts are sharded contiguously (rank g owns [g*E/N, (g+1)*E/N), the first E % N ranks one more); router and
// shared expert are replicated; every rank brings T token rows.  Two exchange schemes:
//
//   SW_EP_REPLICATE  all-gather the rows -> every rank routes all N*T rows identically -> each computes the pairs
//                    of its resident experts -> reduce-scatter of the partial routed sums.  One collective each
//                    way, no index traffic: the scheme for decode-size batches.
//   SW_EP_ALLTOALL   every rank routes ITS OWN rows -> per destination GPU the rows that selected one of its
//                    experts, each row once (deduplicated), go out with their ids and weights (entries of other
//                    GPUs' experts blanked) -> the destination groups what it received by expert, runs its experts
//                    and returns one pre-weighted partial sum per received row -> the owner adds the partial sums
//                    of a row in GPU order.  Row traffic is (GPUs a token reaches) / N of the replicated scheme;
//                    the counts cross once per step (an all-gather of N ints and one host sync to size the
//                    sends).  The scheme for large batches.
//
// The reference has no multi-process layer; its multi-device code moves rows with peer copies,
// c/backend_cuda.cu:1444-1466, and groups per device on the host, c/colibri.c:3506-3607.  Routing ids and the
// dispatch arrays stay bit-identical to the single-GPU result; the cross-GPU sum is in GPU order instead of pure
// rank order (inside the output tolerance).
//
// NCCL is looked up at run time (dlopen of libnccl.so.2): the library itself does not link against it, so hosts
// that never call sw_ep_* need no NCCL.
#include "sw_common.cuh"
#pragma GCC visibility push(default)
#include "../../include/sabrewing_b200.h"
#pragma GCC visibility pop
#include <nccl.h>
#include <dlfcn.h>
#include <string.h>

namespace {
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char *(*GetErrorString)(ncclResult_t);
    bool ok;
};
const NcclApi &nccl() {
    static const NcclApi api = [] {
        NcclApi a{};
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return a;
#define SW_SYM(field, name) a.field = (decltype(a.field))dlsym(h, name); if (!a.field) return a
        SW_SYM(GetUniqueId, "ncclGetUniqueId"); SW_SYM(CommInitRank, "ncclCommInitRank"); SW_SYM(CommDestroy, "ncclCommDestroy");
        SW_SYM(AllGather, "ncclAllGather"); SW_SYM(ReduceScatter, "ncclReduceScatter"); SW_SYM(Send, "ncclSend"); SW_SYM(Recv, "ncclRecv");
        SW_SYM(GroupStart, "ncclGroupStart"); SW_SYM(GroupEnd, "ncclGroupEnd"); SW_SYM(GetErrorString, "ncclGetErrorString");
#undef SW_SYM
        a.ok = true;
        return a;
    }();
    return api;
}
}  // namespace

struct SwEp {
    SwMoeCtx *ctx = nullptr;
    ncclComm_t comm = nullptr;
    int world = 1, rank = 0, dev = 0, num_sms = 0;
    int T = 0, D = 0, K = 0;                 // rows per rank, hidden, top-k the buffers were sized for
    int range_E = -1;                        // expert count the device copy of the shard ranges was made for
    cudaStream_t aux = nullptr;              // the context's second stream: the shared expert runs there
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    void *block = nullptr;                   // one allocation for everything below
    float *X = nullptr, *partial = nullptr, *routed = nullptr, *sendx = nullptr, *ret = nullptr, *sendw = nullptr, *recvw = nullptr;
    int *sendsel = nullptr, *recvsel = nullptr, *send_idx = nullptr, *rank_of = nullptr, *counts = nullptr, *range = nullptr;
    int *h_counts = nullptr;                 // page-locked [world * world]
    float seg_ms[8] = {0};                   // last timed step: segment durations
    cudaEvent_t ev_seg[9] = {nullptr};
};

#define EP_CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { cudaGetLastError(); return sw_fail_text("%s: %s", #call, cudaGetErrorString(e_)); } } while (0)
#define EP_NCCL(call) do { ncclResult_t r_ = (call); if (r_ != ncclSuccess) return sw_fail_text("%s: %s", #call, nccl().GetErrorString(r_)); } while (0)

static void ep_shard(int E, int world, int rank, int *lo, int *cnt) {
    const int base = E / world, rem = E % world;
    *lo = rank * base + (rank < rem ? rank : rem);
    *cnt = base + (rank < rem ? 1 : 0);
}

// ---------------------------------------------------------------------------
// all-to-all scheme: kernels
// ---------------------------------------------------------------------------
// One CTA per destination GPU g: the own rows (ascending) that selected an expert of g get consecutive positions
// in g's send segment.  send_idx[g][pos] = row, rank_of[row][g] = pos (or -1), counts[g] = rows for g.
__global__ void __launch_bounds__(256)
k_ep_plan(const int *__restrict__ sel, int T, int K, const int *__restrict__ range, int world,
          int *__restrict__ send_idx, int *__restrict__ rank_of, int *__restrict__ counts) {
    __shared__ int s_warp[8];
    __shared__ int s_base;
    const int g = blockIdx.x, lo = range[2 * g], hi = lo + range[2 * g + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (int t0 = 0; t0 < T; t0 += 256) {
        const int t = t0 + tid;
        int flag = 0;
        if (t < T) for (int k = 0; k < K; k++) { const int e = sel[t * K + k]; flag |= (e >= lo && e < hi); }
        const unsigned m = __ballot_sync(SW_FULL_MASK, flag);
        if (lane == 0) s_warp[warp] = __popc(m);
        __syncthreads();
        int before = s_base;
        for (int i = 0; i < warp; i++) before += s_warp[i];
        const int pos = before + __popc(m & ((1u << lane) - 1));
        if (t < T) {
            rank_of[t * world + g] = flag ? pos : -1;
            if (flag) send_idx[g * T + pos] = t;
        }
        __syncthreads();
        if (tid == 0) { int tot = 0; for (int i = 0; i < 8; i++) tot += s_warp[i]; s_base += tot; }
        __syncthreads();
    }
    if (tid == 0) counts[g] = s_base;
}

// rows, ids and weights into the send segments: segment g holds counts[g] rows of D floats (capacity T rows); ids of
// experts that do not live on g are blanked
__global__ void __launch_bounds__(256)
k_ep_pack(const float *__restrict__ x, const int *__restrict__ sel, const float *__restrict__ w, const int *__restrict__ send_idx,
          const int *__restrict__ counts, const int *__restrict__ range, int T, int K, int D, int world,
          float *__restrict__ sendx, int *__restrict__ sendsel, float *__restrict__ sendw) {
    const int D4 = D >> 2;
    for (int row = blockIdx.x; row < world * T; row += gridDim.x) {
        const int g = row / T, i = row - g * T;
        if (i >= counts[g]) continue;
        const int t = send_idx[g * T + i];
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)t * D);
        float4 *dst = reinterpret_cast<float4 *>(sendx + (size_t)row * D);
        for (int c = threadIdx.x; c < D4; c += blockDim.x) dst[c] = src[c];
        if (threadIdx.x < K) {
            const int lo = range[2 * g], hi = lo + range[2 * g + 1];
            const int e = sel[t * K + threadIdx.x];
            sendsel[(size_t)row * K + threadIdx.x] = (e >= lo && e < hi) ? e : SW_NO_EXPERT;
            sendw[(size_t)row * K + threadIdx.x] = w[t * K + threadIdx.x];
        }
    }
}

// rows of a receive segment past what the peer sent select nothing
__global__ void __launch_bounds__(256)
k_ep_blank(int *__restrict__ recvsel, const int *__restrict__ all_counts, int rank, int T, int K, int world) {
    const size_t n = (size_t)world * T * K;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(idx / K), g = row / T, i = row - g * T;
        if (i >= all_counts[g * world + rank]) recvsel[idx] = SW_NO_EXPERT;
    }
}

// routed[t] = sum over the GPUs g that row t went to, in GPU order, of the partial sum g returned for it
__global__ void __launch_bounds__(256)
k_ep_sum(const float *__restrict__ ret, const int *__restrict__ rank_of, int T, int D, int world, float *__restrict__ routed) {
    const int D4 = D >> 2;
    const size_t n = (size_t)T * D4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / D4), c = (int)(idx - (size_t)t * D4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int g = 0; g < world; g++) {
            const int pos = rank_of[t * world + g];
            if (pos < 0) continue;
            const float4 v = reinterpret_cast<const float4 *>(ret + ((size_t)g * T + pos) * D)[c];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4 *>(routed)[idx] = acc;
    }
}

// ---------------------------------------------------------------------------
extern "C" int sw_ep_unique_id(void *id128) {
    if (!id128) return sw_fail_text("ep_unique_id: null argument");
    if (!nccl().ok) return sw_fail_text("ep: libnccl.so.2 could not be loaded");
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id size");
    ncclUniqueId id;
    EP_NCCL(nccl().GetUniqueId(&id));
    memcpy(id128, &id, sizeof id);
    return 0;
}

extern "C" void sw_ep_destroy(SwEp *ep) {
    if (!ep) return;
    cudaSetDevice(ep->dev);
    if (ep->comm) nccl().CommDestroy(ep->comm);
    if (ep->block) cudaFree(ep->block);
    if (ep->h_counts) cudaFreeHost(ep->h_counts);
    if (ep->ev_fork) cudaEventDestroy(ep->ev_fork);
    if (ep->ev_join) cudaEventDestroy(ep->ev_join);
    for (cudaEvent_t e : ep->ev_seg) if (e) cudaEventDestroy(e);
    delete ep;
}

extern "C" int sw_ep_create(SwEp **out, SwMoeCtx *ctx, const void *id128, int world, int rank, int rows_per_rank, int D, int K) {
    if (!out) return sw_fail_text("ep_create: null out");
    *out = nullptr;
    if (!ctx || !id128 || world < 1 || rank < 0 || rank >= world || rows_per_rank <= 0 || D <= 0 || (D & 3) || K <= 0 || K > SW_MAX_TOPK)
        return sw_fail_text("ep_create: bad argument");
    if (!nccl().ok) return sw_fail_text("ep: libnccl.so.2 could not be loaded");
    int maxT = 0; void *aux = nullptr;
    SwEp *ep = new SwEp();
    ep->ctx = ctx; ep->world = world; ep->rank = rank; ep->T = rows_per_rank; ep->D = D; ep->K = K;
    sw_ctx_info(ctx, &ep->dev, &ep->num_sms, &maxT, &aux);
    ep->aux = (cudaStream_t)aux;
    if (maxT < world * rows_per_rank) { delete ep; return sw_fail_text("ep_create: the context holds %d rows, the step needs %d (ranks x rows per rank)", maxT, world * rows_per_rank); }
    if (cudaSetDevice(ep->dev) != cudaSuccess) { cudaGetLastError(); delete ep; return sw_fail_text("ep_create: cudaSetDevice failed"); }
    const size_t WT = (size_t)world * rows_per_rank, rowb = (size_t)D * 4;
    auto al = [](size_t n) { return (n + 255) & ~(size_t)255; };
    const size_t sizes[] = {WT * rowb, WT * rowb, (size_t)rows_per_rank * rowb, WT * rowb, WT * rowb,      // X, partial, routed, sendx, ret
                            WT * K * 4, WT * K * 4, WT * K * 4, WT * K * 4,                                  // sendsel, recvsel, sendw, recvw
                            WT * 4, WT * 4, (size_t)(world + world * world) * 4, (size_t)world * 2 * 4};     // send_idx, rank_of, counts, range
    size_t total = 0; for (size_t s : sizes) total += al(s);
    if (cudaMalloc(&ep->block, total) != cudaSuccess) { cudaGetLastError(); ep->block = nullptr; sw_ep_destroy(ep); return sw_fail_text("ep_create: cudaMalloc of %zu bytes failed", total); }
    char *p = (char *)ep->block; int i = 0;
    auto take = [&] { void *q = p; p += al(sizes[i++]); return q; };
    ep->X = (float *)take(); ep->partial = (float *)take(); ep->routed = (float *)take(); ep->sendx = (float *)take(); ep->ret = (float *)take();
    ep->sendsel = (int *)take(); ep->recvsel = (int *)take(); ep->sendw = (float *)take(); ep->recvw = (float *)take();
    ep->send_idx = (int *)take(); ep->rank_of = (int *)take(); ep->counts = (int *)take(); ep->range = (int *)take();
    if (cudaMallocHost((void **)&ep->h_counts, (size_t)world * world * 4) != cudaSuccess ||
        cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ep->ev_join, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); sw_ep_destroy(ep); return sw_fail_text("ep_create: host-side set-up failed"); }
    for (cudaEvent_t &e : ep->ev_seg) if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); e = nullptr; sw_ep_destroy(ep); return sw_fail_text("ep_create: event creation failed"); }
    ncclUniqueId id; memcpy(&id, id128, sizeof id);
    ncclResult_t r = nccl().CommInitRank(&ep->comm, world, id, rank);
    if (r != ncclSuccess) { ep->comm = nullptr; sw_ep_destroy(ep); return sw_fail_text("ncclCommInitRank: %s", nccl().GetErrorString(r)); }
    *out = ep;
    return 0;
}

// One expert-parallel step: out[T,D] += MoE(x[T,D]) for this rank's rows.  `layer` is this rank's shard (expert_lo /
// expert_cnt set, blobs pointing at its first resident expert).  timed != 0 records CUDA events between the segments
// of the step (read them with sw_ep_segments after a stream sync).
extern "C" int sw_ep_forward(SwEp *ep, const SwMoeDesc *d, const SwMoeLayer *L, const float *x, float *out, int T, int scheme, int timed, void *stream) {
    if (!ep || !d || !L || !x || !out) return sw_fail_text("ep_forward: null argument");
    if (T != ep->T || L->D != ep->D || d->topk != ep->K) return sw_fail_text("ep_forward: T, D or top-k differ from what the exchange buffers were created for");
    if (scheme != SW_EP_REPLICATE && scheme != SW_EP_ALLTOALL) return sw_fail_text("ep_forward: unknown scheme %d", scheme);
    cudaStream_t st = (cudaStream_t)stream;
    const int W = ep->world, D = ep->D, K = ep->K;
    const NcclApi &nc = nccl();
    int seg = 0;
    auto mark = [&] { if (timed && seg < 9) cudaEventRecord(ep->ev_seg[seg++], st); };
    const bool has_shared = d->shared_mode != SW_SHARED_NONE;
    // the shared expert needs only this rank's rows: it runs on the context's second stream beside everything else
    if (has_shared) {
        EP_CUDA(cudaEventRecord(ep->ev_fork, st));
        EP_CUDA(cudaStreamWaitEvent(ep->aux, ep->ev_fork, 0));
        if (sw_moe_shared(ep->ctx, d, L, x, T, ep->aux)) return -1;
        EP_CUDA(cudaEventRecord(ep->ev_join, ep->aux));
    }
    mark();
    if (W == 1) {
        if (sw_moe_route(ep->ctx, d, L, x, T, st)) return -1;
        if (sw_moe_experts(ep->ctx, d, L, x, ep->routed, T, st)) return -1;
        mark(); mark(); mark();
    } else if (scheme == SW_EP_REPLICATE) {
        EP_NCCL(nc.AllGather(x, ep->X, (size_t)T * D, ncclFloat32, ep->comm, st));
        mark();
        if (sw_moe_route(ep->ctx, d, L, ep->X, W * T, st)) return -1;
        if (sw_moe_experts(ep->ctx, d, L, ep->X, ep->partial, W * T, st)) return -1;
        mark();
        EP_NCCL(nc.ReduceScatter(ep->partial, ep->routed, (size_t)T * D, ncclFloat32, ncclSum, ep->comm, st));
        mark();
    } else {
        // own rows only: ids and weights of this rank's T rows
        if (sw_moe_route(ep->ctx, d, L, x, T, st)) return -1;
        SwRouting *r = sw_ctx_routing(ep->ctx);
        if (W > 64) return sw_fail_text("ep_forward: more than 64 ranks");
        if (ep->range_E != d->n_experts) {                       // shard ranges of all ranks, uploaded when the layer shape changes
            int h_range[2 * 64];
            for (int g = 0; g < W; g++) ep_shard(d->n_experts, W, g, &h_range[2 * g], &h_range[2 * g + 1]);
            EP_CUDA(cudaMemcpyAsync(ep->range, h_range, (size_t)W * 8, cudaMemcpyHostToDevice, st));
            EP_CUDA(cudaStreamSynchronize(st));
            ep->range_E = d->n_experts;
        }
        k_ep_plan<<<W, 256, 0, st>>>(r->sel, T, K, ep->range, W, ep->send_idx, ep->rank_of, ep->counts);
        sw_count_launch();
        int *all_counts = ep->counts + W;                        // [W][W]: all_counts[src][dst]
        EP_NCCL(nc.AllGather(ep->counts, all_counts, (size_t)W, ncclInt32, ep->comm, st));
        EP_CUDA(cudaMemcpyAsync(ep->h_counts, all_counts, (size_t)W * W * 4, cudaMemcpyDeviceToHost, st));
        int grid = W * T < ep->num_sms * 8 ? W * T : ep->num_sms * 8;
        k_ep_pack<<<grid, 256, 0, st>>>(x, r->sel, r->w, ep->send_idx, ep->counts, ep->range, T, K, D, W, ep->sendx, ep->sendsel, ep->sendw);
        sw_count_launch();
        EP_CUDA(cudaStreamSynchronize(st));                      // the counts size the sends: the one host sync of a step
        EP_CUDA(cudaGetLastError());
        const int *hc = ep->h_counts;
        mark();
        EP_NCCL(nc.GroupStart());
        for (int g = 0; g < W; g++) {
            const size_t ns = (size_t)hc[ep->rank * W + g], nr = (size_t)hc[g * W + ep->rank], off = (size_t)g * T;
            if (g == ep->rank) {                                 // rows for the own experts stay here
                if (ns) {
                    EP_CUDA(cudaMemcpyAsync(ep->X + off * D, ep->sendx + off * D, ns * D * 4, cudaMemcpyDeviceToDevice, st));
                    EP_CUDA(cudaMemcpyAsync(ep->recvsel + off * K, ep->sendsel + off * K, ns * K * 4, cudaMemcpyDeviceToDevice, st));
                    EP_CUDA(cudaMemcpyAsync(ep->recvw + off * K, ep->sendw + off * K, ns * K * 4, cudaMemcpyDeviceToDevice, st));
                }
                continue;
            }
            if (ns) {
                EP_NCCL(nc.Send(ep->sendx + off * D, ns * D, ncclFloat32, g, ep->comm, st));
                EP_NCCL(nc.Send(ep->sendsel + off * K, ns * K, ncclInt32, g, ep->comm, st));
                EP_NCCL(nc.Send(ep->sendw + off * K, ns * K, ncclFloat32, g, ep->comm, st));
            }
            if (nr) {
                EP_NCCL(nc.Recv(ep->X + off * D, nr * D, ncclFloat32, g, ep->comm, st));
                EP_NCCL(nc.Recv(ep->recvsel + off * K, nr * K, ncclInt32, g, ep->comm, st));
                EP_NCCL(nc.Recv(ep->recvw + off * K, nr * K, ncclFloat32, g, ep->comm, st));
            }
        }
        EP_NCCL(nc.GroupEnd());
        k_ep_blank<<<ep->num_sms, 256, 0, st>>>(ep->recvsel, all_counts, ep->rank, T, K, W);
        sw_count_launch();
        mark();
        if (sw_moe_experts_routed(ep->ctx, d, L, ep->X, ep->recvsel, ep->recvw, ep->partial, W * T, st)) return -1;
        mark();
        EP_NCCL(nc.GroupStart());
        for (int g = 0; g < W; g++) {
            const size_t ns = (size_t)hc[g * W + ep->rank], nr = (size_t)hc[ep->rank * W + g], off = (size_t)g * T;
            if (g == ep->rank) {
                if (ns) EP_CUDA(cudaMemcpyAsync(ep->ret + off * D, ep->partial + off * D, ns * D * 4, cudaMemcpyDeviceToDevice, st));
                continue;
            }
            if (ns) EP_NCCL(nc.Send(ep->partial + off * D, ns * D, ncclFloat32, g, ep->comm, st));
            if (nr) EP_NCCL(nc.Recv(ep->ret + off * D, nr * D, ncclFloat32, g, ep->comm, st));
        }
        EP_NCCL(nc.GroupEnd());
        {
            size_t n = (size_t)T * (D / 4);
            long long g2 = (long long)((n + 255) / 256);
            if (g2 > (long long)ep->num_sms * 16) g2 = (long long)ep->num_sms * 16;
            k_ep_sum<<<(unsigned)g2, 256, 0, st>>>(ep->ret, ep->rank_of, T, D, W, ep->routed);
            sw_count_launch();
        }
        mark();
    }
    if (has_shared) EP_CUDA(cudaStreamWaitEvent(st, ep->ev_join, 0));
    if (sw_moe_finish(ep->ctx, d, L, x, ep->routed, out, T, st)) return -1;
    mark();
    EP_CUDA(cudaGetLastError());
    return 0;
}

// ms of the segments of the last step run with timed != 0 (synchronise the stream first): for SW_EP_REPLICATE
// {all-gather, route + experts, reduce-scatter, finish}, for SW_EP_ALLTOALL {route + plan + pack + count exchange,
// rows out, experts, partial sums back + add, finish}.  Returns the number of segments written (<= 8).
extern "C" int sw_ep_segments(SwEp *ep, float *ms, int scheme) {
    if (!ep || !ms) return sw_fail_text("ep_segments: null argument");
    const int n = scheme == SW_EP_ALLTOALL ? 5 : 4;
    for (int i = 0; i < n; i++) {
        if (cudaEventElapsedTime(&ms[i], ep->ev_seg[i], ep->ev_seg[i + 1]) != cudaSuccess) { cudaGetLastError(); return sw_fail_text("ep_segments: no timed step recorded"); }
    }
    return n;
}
