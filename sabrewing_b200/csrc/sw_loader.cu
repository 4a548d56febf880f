// Container loader: one MoE layer of a Laguna int4 snapshot straight from its safetensors files into device memory.
//
// Layout read (the reference's container, docs/laguna.md:34-42, written by c/tools/convert_laguna_int4.py and loaded by
// c/laguna.c:410-446 through c/st.h):
//   model.layers.{i}.mlp.gate.weight                          router, F32 (or BF16) [E, D]
//   model.layers.{i}.mlp.experts.e_score_correction_bias      F32 [E]
//   model.layers.{i}.mlp.experts.gate_up_proj (+ .qs)         U8 [E*2I, D/2] packed int4, gate rows then up rows per
//                                                            expert; F32 [E*2I] row scales
//   model.layers.{i}.mlp.experts.down_proj (+ .qs)            U8 [E*D, I/2]; F32 [E*D]
//   model.layers.{i}.mlp.shared_expert.{gate,up,down}_proj.weight   BF16 [SI, D], [SI, D], [D, SI]
// A safetensors file is an 8-byte little-endian header length, a JSON header (name -> dtype, shape, data_offsets) and
// the raw tensor bytes.  The header is scanned for the names above only (no general JSON tree is built).  Tensor bytes
// go file -> page-locked staging block -> device in chunks, two chunks in flight; nothing is kept on the host.  With
// expert_cnt > 0 only the rows of experts [expert_lo, expert_lo + expert_cnt) are read (expert-parallel shard).
#include "sw_common.cuh"
#pragma GCC visibility push(default)
#include "../../include/sabrewing_b200.h"
#pragma GCC visibility pop
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>
#include <fcntl.h>
#include <unistd.h>
#include <dirent.h>
#include <sys/stat.h>

namespace {
struct StTensor { int fd; long long off, nbytes; std::string dtype; std::vector<long long> shape; };
struct StFile { int fd; std::string header; long long data0; };

#define LD_FAIL(...) do { sw_fail_text(__VA_ARGS__); return -1; } while (0)

int open_file(const std::string &path, StFile *f) {
    f->fd = open(path.c_str(), O_RDONLY);
    if (f->fd < 0) LD_FAIL("loader: cannot open %s", path.c_str());
    unsigned char len8[8];
    if (pread(f->fd, len8, 8, 0) != 8) { close(f->fd); LD_FAIL("loader: %s is too short", path.c_str()); }
    unsigned long long n = 0;
    for (int i = 7; i >= 0; i--) n = (n << 8) | len8[i];
    if (n < 2 || n > (512ull << 20)) { close(f->fd); LD_FAIL("loader: %s declares a header of %llu bytes", path.c_str(), n); }
    f->header.resize((size_t)n);
    if (pread(f->fd, &f->header[0], (size_t)n, 8) != (ssize_t)n) { close(f->fd); LD_FAIL("loader: short header in %s", path.c_str()); }
    f->data0 = 8 + (long long)n;
    return 0;
}
// finds "name":{...} in a header and reads dtype, shape, data_offsets out of the object
bool find_tensor(const StFile &f, const std::string &name, StTensor *t) {
    const std::string key = "\"" + name + "\"";
    size_t p = 0;
    for (;;) {
        p = f.header.find(key, p);
        if (p == std::string::npos) return false;
        size_t q = p + key.size();
        while (q < f.header.size() && (f.header[q] == ' ' || f.header[q] == '\n' || f.header[q] == '\t')) q++;
        if (q < f.header.size() && f.header[q] == ':') { p = q + 1; break; }
        p += key.size();                                          // the name occurred as a value, not as a key
    }
    const size_t ob = f.header.find('{', p), oe = ob == std::string::npos ? ob : f.header.find('}', ob);
    if (ob == std::string::npos || oe == std::string::npos) return false;
    const std::string obj = f.header.substr(ob, oe - ob + 1);
    auto after = [&](const char *k) -> size_t { size_t a = obj.find(k); return a == std::string::npos ? a : obj.find(':', a) + 1; };
    size_t a = after("\"dtype\"");
    if (a == std::string::npos) return false;
    size_t q0 = obj.find('"', a), q1 = q0 == std::string::npos ? q0 : obj.find('"', q0 + 1);
    if (q1 == std::string::npos) return false;
    t->dtype = obj.substr(q0 + 1, q1 - q0 - 1);
    auto numbers = [&](const char *k, std::vector<long long> *out) -> bool {
        size_t b = after(k);
        if (b == std::string::npos) return false;
        size_t lb = obj.find('[', b), rb = lb == std::string::npos ? lb : obj.find(']', lb);
        if (rb == std::string::npos) return false;
        out->clear();
        const char *s = obj.c_str() + lb + 1, *e = obj.c_str() + rb;
        while (s < e) {
            while (s < e && (*s < '0' || *s > '9')) s++;
            if (s >= e) break;
            char *end; out->push_back(strtoll(s, &end, 10)); s = end;
        }
        return true;
    };
    std::vector<long long> offs;
    if (!numbers("\"shape\"", &t->shape) || !numbers("\"data_offsets\"", &offs) || offs.size() != 2 || offs[1] < offs[0]) return false;
    t->fd = f.fd; t->off = f.data0 + offs[0]; t->nbytes = offs[1] - offs[0];
    return true;
}

struct Stager {                       // file -> page-locked block -> device, two chunks in flight
    static const size_t CHUNK = 32u << 20;
    char *h[2] = {nullptr, nullptr}; cudaEvent_t ev[2] = {nullptr, nullptr}; cudaStream_t st = nullptr; int turn = 0;
    int init() {
        for (int i = 0; i < 2; i++) if (cudaMallocHost((void **)&h[i], CHUNK) != cudaSuccess || cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return -1; }
        return cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess ? 0 : (cudaGetLastError(), -1);
    }
    int copy(void *dst, int fd, long long off, long long n) {
        for (long long done = 0; done < n;) {
            const size_t m = (size_t)((n - done) < (long long)CHUNK ? (n - done) : (long long)CHUNK);
            if (cudaEventSynchronize(ev[turn]) != cudaSuccess) { cudaGetLastError(); return -1; }      // the block's previous copy has left it
            for (size_t got = 0; got < m;) {
                const ssize_t r = pread(fd, h[turn] + got, m - got, off + done + (long long)got);
                if (r <= 0) return -1;
                got += (size_t)r;
            }
            if (cudaMemcpyAsync((char *)dst + done, h[turn], m, cudaMemcpyHostToDevice, st) != cudaSuccess || cudaEventRecord(ev[turn], st) != cudaSuccess) { cudaGetLastError(); return -1; }
            done += (long long)m; turn ^= 1;
        }
        return 0;
    }
    ~Stager() {
        if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
        for (int i = 0; i < 2; i++) { if (h[i]) cudaFreeHost(h[i]); if (ev[i]) cudaEventDestroy(ev[i]); }
    }
};
}  // namespace

struct SwLoadedLayer { int dev; std::vector<void *> blocks; };

extern "C" void sw_layer_free(SwLoadedLayer *h) {
    if (!h) return;
    cudaSetDevice(h->dev);
    for (void *p : h->blocks) cudaFree(p);
    delete h;
}

// path: a .safetensors file or a directory of them.  On success *layer describes device-resident weights owned by
// *handle (free with sw_layer_free), and n_experts / has_bias report what the container held.
extern "C" int sw_layer_load(const char *path, int layer_index, int dev, int expert_lo, int expert_cnt,
                             SwMoeLayer *layer, int *n_experts, SwLoadedLayer **handle) {
    if (!path || !layer || !handle || layer_index < 0) LD_FAIL("loader: bad argument");
    *handle = nullptr;
    std::vector<std::string> paths;
    struct stat sb;
    if (stat(path, &sb) != 0) LD_FAIL("loader: %s does not exist", path);
    if (S_ISDIR(sb.st_mode)) {
        DIR *d = opendir(path);
        if (!d) LD_FAIL("loader: cannot list %s", path);
        while (dirent *e = readdir(d)) {
            const std::string n = e->d_name;
            if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) paths.push_back(std::string(path) + "/" + n);
        }
        closedir(d);
    } else paths.push_back(path);
    if (paths.empty()) LD_FAIL("loader: no .safetensors file under %s", path);
    std::vector<StFile> files(paths.size());
    size_t nopen = 0;
    auto close_all = [&] { for (size_t i = 0; i < nopen; i++) close(files[i].fd); };
    for (; nopen < paths.size(); nopen++) if (open_file(paths[nopen], &files[nopen])) { close_all(); return -1; }
    char base[128]; snprintf(base, sizeof base, "model.layers.%d.mlp.", layer_index);
    auto get = [&](const char *suffix, StTensor *t) { for (const StFile &f : files) if (find_tensor(f, std::string(base) + suffix, t)) return true; return false; };

    StTensor router, ebias, guq, gus, dnq, dns, sg, su, sd;
    const bool has_bias = get("experts.e_score_correction_bias", &ebias);
    if (!get("gate.weight", &router) || !get("experts.gate_up_proj", &guq) || !get("experts.gate_up_proj.qs", &gus) ||
        !get("experts.down_proj", &dnq) || !get("experts.down_proj.qs", &dns)) { close_all(); LD_FAIL("loader: layer %d is not an int4 MoE layer of this container (a tensor is missing)", layer_index); }
    const bool has_shared = get("shared_expert.gate_proj.weight", &sg) && get("shared_expert.up_proj.weight", &su) && get("shared_expert.down_proj.weight", &sd);
    if (router.shape.size() != 2 || guq.shape.size() != 2 || dnq.shape.size() != 2 || guq.dtype != "U8" || dnq.dtype != "U8" ||
        gus.dtype != "F32" || dns.dtype != "F32" || (router.dtype != "F32" && router.dtype != "BF16")) { close_all(); LD_FAIL("loader: unexpected dtype or rank in layer %d", layer_index); }
    const long long E = router.shape[0], D = router.shape[1];
    const long long I = E > 0 ? guq.shape[0] / (2 * E) : 0;
    if (E <= 0 || D <= 0 || I <= 0 || guq.shape[0] != 2 * E * I || guq.shape[1] * 2 != D || dnq.shape[0] != E * D || dnq.shape[1] * 2 != I ||
        gus.nbytes != 2 * E * I * 4 || dns.nbytes != E * D * 4 || guq.nbytes != 2 * E * I * (D / 2) || dnq.nbytes != E * D * (I / 2) ||
        router.nbytes != E * D * (router.dtype == "F32" ? 4 : 2) || (has_bias && ebias.nbytes != E * 4)) { close_all(); LD_FAIL("loader: inconsistent shapes in layer %d", layer_index); }
    long long SI = 0;
    if (has_shared) {
        SI = sg.shape.size() == 2 ? sg.shape[0] : 0;
        if (SI <= 0 || sg.dtype != "BF16" || su.dtype != "BF16" || sd.dtype != "BF16" || sg.nbytes != SI * D * 2 || su.nbytes != SI * D * 2 || sd.nbytes != D * SI * 2) { close_all(); LD_FAIL("loader: unexpected shared-expert tensors in layer %d", layer_index); }
    }
    long long lo = 0, cnt = E;
    if (expert_cnt > 0) { lo = expert_lo; cnt = expert_cnt; if (lo < 0 || lo + cnt > E) { close_all(); LD_FAIL("loader: expert range [%lld, %lld) outside [0, %lld)", lo, lo + cnt, E); } }

    if (cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); close_all(); LD_FAIL("loader: cudaSetDevice(%d) failed", dev); }
    Stager stg;
    SwLoadedLayer *h = new SwLoadedLayer{dev, {}};
    auto fail = [&](const char *what) { sw_layer_free(h); close_all(); sw_fail_text("loader: %s failed", what); return -1; };
    if (stg.init()) return fail("staging set-up");
    auto put = [&](const StTensor &t, long long off, long long n, void **out) -> int {
        void *d = nullptr;
        if (cudaMalloc(&d, (size_t)n) != cudaSuccess) { cudaGetLastError(); return -1; }
        h->blocks.push_back(d);
        *out = d;
        return stg.copy(d, t.fd, t.off + off, n);
    };
    void *p_router, *p_bias = nullptr, *p_guq, *p_gus, *p_dnq, *p_dns, *p_sg = nullptr, *p_su = nullptr, *p_sd = nullptr;
    const long long gurow = D / 2, dnrow = I / 2;
    if (put(router, 0, router.nbytes, &p_router) || (has_bias && put(ebias, 0, ebias.nbytes, &p_bias)) ||
        put(guq, lo * 2 * I * gurow, cnt * 2 * I * gurow, &p_guq) || put(gus, lo * 2 * I * 4, cnt * 2 * I * 4, &p_gus) ||
        put(dnq, lo * D * dnrow, cnt * D * dnrow, &p_dnq) || put(dns, lo * D * 4, cnt * D * 4, &p_dns) ||
        (has_shared && (put(sg, 0, sg.nbytes, &p_sg) || put(su, 0, su.nbytes, &p_su) || put(sd, 0, sd.nbytes, &p_sd)))) return fail("reading or uploading a tensor");
    if (cudaStreamSynchronize(stg.st) != cudaSuccess) { cudaGetLastError(); return fail("upload"); }
    close_all();
    memset(layer, 0, sizeof *layer);
    layer->D = (int)D; layer->I = (int)I; layer->SI = (int)SI;
    layer->router_dtype = router.dtype == "F32" ? SW_DTYPE_F32 : SW_DTYPE_BF16;
    layer->router_w = p_router; layer->corr_bias = (const float *)p_bias; layer->logit_bias = nullptr;
    layer->gu_q = p_guq; layer->gu_s = (const float *)p_gus; layer->dn_q = p_dnq; layer->dn_s = (const float *)p_dns;
    layer->sh_gate = p_sg; layer->sh_up = p_su; layer->sh_down = p_sd;
    layer->expert_lo = expert_cnt > 0 ? (int)lo : 0; layer->expert_cnt = expert_cnt > 0 ? (int)cnt : 0; layer->gs = 0;
    if (n_experts) *n_experts = (int)E;
    *handle = h;
    return 0;
}
