// The vocab-sharded sampling step as one C-ABI call that owns its collectives.
//
// A tensor-parallel LM head leaves every GPU with a contiguous slice of each row's logits. The
// step is the four stage functions of molla_sample.cu with two all-gathers between them, all
// enqueued by this one call: a host that binds C and has no NCCL binding of its own (the
// reference loads its C libraries the way src/molla/tls/openssl.mojo:53-139 does) drives it
// with a communicator handle this library created for it. NCCL is loaded at run time
// (dlopen of libnccl.so.2), so the library still loads on a machine without it; peers' data
// only ever arrives through NCCL into this GPU's own memory.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/molla_sample.h"

namespace {

// the few NCCL entry points used, by their public C signatures (nccl.h)
typedef struct { char internal[128]; } NcclUniqueId;
typedef int (*fn_get_unique_id)(NcclUniqueId *);
typedef int (*fn_comm_init_rank)(void **, int, NcclUniqueId, int);
typedef int (*fn_comm_destroy)(void *);
typedef int (*fn_all_gather)(const void *, void *, size_t, int /*ncclDataType_t*/, void *, cudaStream_t);
typedef const char *(*fn_error_string)(int);
constexpr int NCCL_INT8 = 0;  // ncclInt8 / ncclChar: bytes are all that is ever sent

struct Nccl {
    void *handle = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_error_string error_string = nullptr;
};

thread_local char s_err[512] = "";

int failed(int code, const char *fmt, const char *detail = "") {
    snprintf(s_err, sizeof(s_err), fmt, detail);
    return code;
}

Nccl *nccl() {
    static Nccl n;
    static bool tried = false;
    if (!tried) {
        tried = true;
        const char *path = getenv("MOLLA_LIBNCCL");  // same pattern as MOLLA_LIBSSL in the reference
        n.handle = dlopen(path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (n.handle) {
            n.get_unique_id = (fn_get_unique_id)dlsym(n.handle, "ncclGetUniqueId");
            n.comm_init_rank = (fn_comm_init_rank)dlsym(n.handle, "ncclCommInitRank");
            n.comm_destroy = (fn_comm_destroy)dlsym(n.handle, "ncclCommDestroy");
            n.all_gather = (fn_all_gather)dlsym(n.handle, "ncclAllGather");
            n.error_string = (fn_error_string)dlsym(n.handle, "ncclGetErrorString");
        }
    }
    if (!n.handle || !n.get_unique_id || !n.comm_init_rank || !n.comm_destroy || !n.all_gather) return nullptr;
    return &n;
}

inline size_t al256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Layout {
    size_t ws_local, ws_global, summary, gathered, global4, lst, count, counts_all, send, recv, total;
};

Layout layout(int B, int Vl, int Vg, int world, int list_cap) {
    Layout L;
    const int words = molla_sample_shard_summary_words();
    size_t o = 0;
    L.ws_local = o; o += al256((size_t)molla_sample_workspace_bytes(B, Vl, 0));
    L.ws_global = o; o += al256((size_t)molla_sample_workspace_bytes(B, Vg, 0));
    L.summary = o; o += al256((size_t)B * words * 4);
    L.gathered = o; o += al256((size_t)world * B * words * 4);
    L.global4 = o; o += al256((size_t)B * 16);
    L.lst = o; o += al256((size_t)B * list_cap * 8);
    L.count = o; o += al256((size_t)B * 4);
    L.counts_all = o; o += al256((size_t)world * B * 4);
    L.send = o; o += al256((size_t)B * list_cap * 8);
    L.recv = o; o += al256((size_t)world * B * list_cap * 8);
    L.total = o;
    return L;
}

}  // namespace

extern "C" {

const char *molla_sample_sharded_last_error(void) { return s_err; }

int32_t molla_sample_nccl_unique_id(uint8_t *out128) {
    s_err[0] = 0;
    Nccl *n = nccl();
    if (!n) return failed(MOLLA_ERR_CUDA, "libnccl.so.2 could not be loaded (set MOLLA_LIBNCCL to its path)%s");
    if (!out128) return failed(MOLLA_ERR_ARGUMENT, "no room for the id%s");
    NcclUniqueId id;
    const int rc = n->get_unique_id(&id);
    if (rc != 0) return failed(MOLLA_ERR_CUDA, "ncclGetUniqueId: %s", n->error_string ? n->error_string(rc) : "failed");
    memcpy(out128, &id, 128);
    return MOLLA_OK;
}

int32_t molla_sample_nccl_comm_create(const uint8_t *id128, int32_t rank, int32_t world, void **comm_out) {
    s_err[0] = 0;
    Nccl *n = nccl();
    if (!n) return failed(MOLLA_ERR_CUDA, "libnccl.so.2 could not be loaded (set MOLLA_LIBNCCL to its path)%s");
    if (!id128 || !comm_out || world < 1 || rank < 0 || rank >= world) return failed(MOLLA_ERR_ARGUMENT, "bad communicator arguments%s");
    NcclUniqueId id;
    memcpy(&id, id128, 128);
    void *comm = nullptr;
    const int rc = n->comm_init_rank(&comm, world, id, rank);
    if (rc != 0) return failed(MOLLA_ERR_CUDA, "ncclCommInitRank: %s", n->error_string ? n->error_string(rc) : "failed");
    *comm_out = comm;
    return MOLLA_OK;
}

int32_t molla_sample_nccl_comm_destroy(void *comm) {
    s_err[0] = 0;
    Nccl *n = nccl();
    if (!n || !comm) return failed(MOLLA_ERR_ARGUMENT, "no communicator%s");
    return n->comm_destroy(comm) == 0 ? MOLLA_OK : failed(MOLLA_ERR_CUDA, "ncclCommDestroy failed%s");
}

int64_t molla_sample_sharded_workspace_bytes(int32_t B, int32_t V_local, int32_t V_global, int32_t world, int32_t list_cap) {
    s_err[0] = 0;
    if (B < 0 || V_local <= 0 || V_global < V_local || world < 1 || world > 16 || list_cap < 1)
        return failed(MOLLA_ERR_ARGUMENT, "bad shape for the sharded workspace query%s");
    return (int64_t)layout(B, V_local, V_global, world, list_cap).total;
}

int32_t molla_sample_sharded_step(void *comm, int32_t rank, int32_t world, const float *d_logits, int64_t row_stride,
                                  int32_t B, int32_t V_local, int32_t col0, int32_t V_global,
                                  const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
                                  const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
                                  const float *d_frequency_penalty, const float *d_presence_penalty,
                                  const uint8_t *d_window_on, const int64_t *d_hist, const int32_t *d_hist_off,
                                  const int64_t *d_bias_ids, const float *d_bias_vals, const int32_t *d_bias_off,
                                  const uint64_t *d_seed, const uint64_t *d_drawn, int32_t list_cap,
                                  void *d_workspace, int64_t workspace_bytes, void *stream, int32_t *d_tokens,
                                  uint32_t *d_row_status, float *d_diag, int64_t *wire_bytes) {
    s_err[0] = 0;
    Nccl *n = nccl();
    if (!n) return failed(MOLLA_ERR_CUDA, "libnccl.so.2 could not be loaded (set MOLLA_LIBNCCL to its path)%s");
    if (!comm || world < 1 || world > 16 || rank < 0 || rank >= world)
        return failed(MOLLA_ERR_ARGUMENT, "a communicator of at most 16 ranks and this rank's place in it are required%s");
    if (!d_logits || !d_tokens || !d_row_status || B < 0 || V_local <= 0 || list_cap < 1 || col0 < 0 ||
        (long long)col0 + V_local > V_global)
        return failed(MOLLA_ERR_ARGUMENT, "bad arguments to the sharded step%s");
    if (list_cap > V_local) list_cap = V_local;
    const Layout L = layout(B, V_local, V_global, world, list_cap);
    if (!d_workspace || workspace_bytes < (int64_t)L.total) return failed(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    char *w = (char *)d_workspace;
    cudaStream_t st = (cudaStream_t)stream;
    const int words = molla_sample_shard_summary_words();
    auto relay = [&](int rc) { if (rc != MOLLA_OK) snprintf(s_err, sizeof(s_err), "%s", molla_sample_last_error()); return rc; };
    auto gather = [&](const void *src, void *dst, size_t bytes) -> int {
        const int rc = n->all_gather(src, dst, bytes, NCCL_INT8, comm, st);
        return rc == 0 ? MOLLA_OK : failed(MOLLA_ERR_CUDA, "ncclAllGather: %s", n->error_string ? n->error_string(rc) : "failed");
    };
    int rc;
    // 1. what the other shards need to know about this slice, to everybody
    rc = relay(molla_sample_shard_stage_a(d_logits, row_stride, B, V_local, col0, V_global, d_temperature, d_top_k, d_top_p,
                                          d_min_p, d_typical_p, d_repeat_penalty, d_frequency_penalty, d_presence_penalty,
                                          d_window_on, d_hist, d_hist_off, d_bias_ids, d_bias_vals, d_bias_off,
                                          w + L.ws_local, (int64_t)(L.ws_global - L.ws_local), stream, (float *)(w + L.summary)));
    if (rc != MOLLA_OK) return rc;
    if ((rc = gather(w + L.summary, w + L.gathered, (size_t)B * words * 4)) != MOLLA_OK) return rc;
    // 2. the row maxima and head thresholds; greedy rows are answered here
    rc = relay(molla_sample_shard_merge(B, V_global, world, rank, d_temperature, d_top_k, (const float *)(w + L.gathered), stream,
                                        (float *)(w + L.global4), d_tokens, d_row_status));
    if (rc != MOLLA_OK) return rc;
    // 3. this slice's list against the row's maximum
    rc = relay(molla_sample_shard_stage_b(d_logits, row_stride, B, V_local, col0, V_global, d_temperature, d_top_k, d_top_p,
                                          d_min_p, d_typical_p, d_repeat_penalty, d_frequency_penalty, d_presence_penalty,
                                          d_window_on, d_hist, d_hist_off, d_bias_ids, d_bias_vals, d_bias_off,
                                          (const float *)(w + L.global4), list_cap, w + L.ws_local,
                                          (int64_t)(L.ws_global - L.ws_local), stream, (uint64_t *)(w + L.lst), (int32_t *)(w + L.count)));
    if (rc != MOLLA_OK) return rc;
    // 4. the counts first: only as many entries per row as the longest list anywhere has go on the wire
    if ((rc = gather(w + L.count, w + L.counts_all, (size_t)B * 4)) != MOLLA_OK) return rc;
    static thread_local int32_t *h_counts = nullptr;
    static thread_local size_t h_cap = 0;
    const size_t nc = (size_t)world * B;
    if (h_cap < nc) {
        if (h_counts) cudaFreeHost(h_counts);
        h_counts = nullptr; h_cap = 0;
        if (cudaMallocHost((void **)&h_counts, nc * 4) != cudaSuccess) return failed(MOLLA_ERR_CUDA, "no pinned memory for the list counts%s");
        h_cap = nc;
    }
    cudaError_t e = cudaMemcpyAsync(h_counts, w + L.counts_all, nc * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return failed(MOLLA_ERR_CUDA, "reading the list counts failed: %s", cudaGetErrorString(e));
    int maxc = 1;
    for (size_t i = 0; i < nc; i++) maxc = h_counts[i] > maxc ? h_counts[i] : maxc;
    if (maxc > list_cap) maxc = list_cap;
    e = cudaMemcpy2DAsync(w + L.send, (size_t)maxc * 8, w + L.lst, (size_t)list_cap * 8, (size_t)maxc * 8, (size_t)B,
                          cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return failed(MOLLA_ERR_CUDA, "packing the lists failed: %s", cudaGetErrorString(e));
    if ((rc = gather(w + L.send, w + L.recv, (size_t)B * maxc * 8)) != MOLLA_OK) return rc;
    // 5. the shards' lists in column order are the unsharded row's list: the rest as on one GPU
    rc = relay(molla_sample_shard_stage_c(B, V_global, d_temperature, d_top_k, d_top_p, d_min_p, d_typical_p, d_seed, d_drawn,
                                          (const float *)(w + L.global4), world, maxc, (const uint64_t *)(w + L.recv),
                                          (const int32_t *)(w + L.counts_all), w + L.ws_global, (int64_t)(L.summary - L.ws_global),
                                          stream, d_tokens, d_row_status, d_diag));
    if (rc != MOLLA_OK) return rc;
    if (wire_bytes) {
        const int64_t sent = (int64_t)B * words * 4 + (int64_t)B * 4 + (int64_t)B * maxc * 8;
        wire_bytes[0] = sent;                 // what this rank contributes to the three all-gathers
        wire_bytes[1] = sent * world;         // what it ends up holding
        wire_bytes[2] = maxc;                 // entries per row that went on the wire
    }
    return MOLLA_OK;
}

}  // extern "C"
