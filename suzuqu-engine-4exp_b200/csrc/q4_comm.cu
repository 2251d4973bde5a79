/*
 * The collective form of the record exchange of a sequence-sharded decode: every rank all-gathers its
 * (m, l, acc) records over NCCL and merges them (gqa_dec_comb_k's arithmetic, src/q4_rocm.cu:6968-7012,
 * taken across GPUs; the reference itself runs one GPU and has no collective).  The communicator is
 * built from a unique id that the HOST passes along by whatever channel it has (a file, a socket, its own
 * launcher), one process per GPU.
 *
 * NCCL is looked up at run time (dlopen of libnccl.so.2, the copy already in the process if there is one):
 * the library has no link-time dependency on it, and a host that never calls q4_gpu_comm_* never loads it.
 * The in-kernel exchange (q4_gpu_kv_decode_xchg) is the faster path on one NVLink node; this one is what a
 * host with its own NCCL set-up, or more than one node, uses.
 */
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "q4_internal.h"

namespace {

struct NcclId { char bytes[128]; };                    /* ncclUniqueId */
typedef void *NcclComm;
typedef int (*GetUniqueIdFn)(NcclId *);
typedef int (*CommInitRankFn)(NcclComm *, int, NcclId, int);
typedef int (*CommDestroyFn)(NcclComm);
typedef int (*AllGatherFn)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
typedef const char *(*GetErrorStringFn)(int);
constexpr int NCCL_FLOAT32 = 7;                        /* ncclFloat32 */

struct Nccl {
    void *h = nullptr;
    GetUniqueIdFn get_id = nullptr;
    CommInitRankFn init_rank = nullptr;
    CommDestroyFn destroy = nullptr;
    AllGatherFn all_gather = nullptr;
    GetErrorStringFn err = nullptr;
    bool tried = false, ok = false;
} g_nccl;

bool nccl_load() {
    Nccl &N = g_nccl;
    if (N.tried) return N.ok;
    N.tried = true;
    const char *names[] = {getenv("Q4_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n) continue;
        N.h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (N.h) break;
    }
    if (!N.h) return q4i_fail(Q4E_ARG, "comm: libnccl.so.2 not found (set Q4_NCCL_LIB)");
    N.get_id = (GetUniqueIdFn)dlsym(N.h, "ncclGetUniqueId");
    N.init_rank = (CommInitRankFn)dlsym(N.h, "ncclCommInitRank");
    N.destroy = (CommDestroyFn)dlsym(N.h, "ncclCommDestroy");
    N.all_gather = (AllGatherFn)dlsym(N.h, "ncclAllGather");
    N.err = (GetErrorStringFn)dlsym(N.h, "ncclGetErrorString");
    N.ok = N.get_id && N.init_rank && N.destroy && N.all_gather;
    if (!N.ok) return q4i_fail(Q4E_ARG, "comm: the NCCL library lacks an entry point");
    return true;
}
bool nccl_check(int rc, const char *what) {
    if (rc == 0) return true;
    g_q4.err_h |= Q4E_CUDA;
    fprintf(stderr, "q4 gpu: %s: %s\n", what, g_nccl.err ? g_nccl.err(rc) : "NCCL error");
    return false;
}

}  // namespace

struct q4_gpu_comm {
    NcclComm comm;
    uint32_t rank, world;
};

extern "C" bool q4_gpu_comm_unique_id(void *id128) {
    if (!id128) return false;
    if (!nccl_load()) return false;
    NcclId id;
    if (!nccl_check(g_nccl.get_id(&id), "comm: ncclGetUniqueId")) return false;
    memcpy(id128, id.bytes, sizeof(id.bytes));
    return true;
}

extern "C" q4_gpu_comm *q4_gpu_comm_create(const void *id128, uint32_t rank, uint32_t world) {
    if (!g_q4.ok) { q4i_fail(Q4E_INIT, "comm_create: library not initialised"); return nullptr; }
    if (!id128 || !world || rank >= world || g_q4.capturing) { q4i_fail(Q4E_ARG, "comm_create: bad argument"); return nullptr; }
    if (!nccl_load()) return nullptr;
    q4_gpu_comm *c = (q4_gpu_comm *)calloc(1, sizeof(q4_gpu_comm));
    if (!c) return nullptr;
    NcclId id;
    memcpy(id.bytes, id128, sizeof(id.bytes));
    if (!nccl_check(g_nccl.init_rank(&c->comm, (int)world, id, (int)rank), "comm_create: ncclCommInitRank")) {
        free(c);
        return nullptr;
    }
    c->rank = rank;
    c->world = world;
    return c;
}

extern "C" void q4_gpu_comm_destroy(q4_gpu_comm *c) {
    if (!c) return;
    if (c->comm && g_nccl.ok) (void)g_nccl.destroy(c->comm);
    free(c);
}

extern "C" bool q4_gpu_comm_allgather_merge(q4_gpu_comm *c, const float *part, float *parts_all, uint32_t n_head, uint32_t hd,
                                            const float *gate, float *out) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "comm_allgather_merge: library not initialised");
    Q4_REQUIRE(c && part && parts_all && out && n_head && hd, "comm_allgather_merge: null/zero argument");
    const size_t n = (size_t)n_head * (hd + 2);
    if (!nccl_check(g_nccl.all_gather(part, parts_all, n, NCCL_FLOAT32, c->comm, g_q4.stream), "comm: ncclAllGather")) return false;
    return q4_gpu_lse_merge(parts_all, c->world, n_head, hd, gate, out);
}
