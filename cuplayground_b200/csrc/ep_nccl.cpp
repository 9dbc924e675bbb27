// Expert-parallel all-to-all on NCCL send/recv groups.
//
// Replaces the reference's device-initiated NVSHMEM exchange (auditorium/overlap.cuh:94-153:
// nvshmemx_putmem_signal_nbi_block to the peer's symmetric heap, then an unbounded nvshmem_signal_wait_until spin)
// and its bootstrap (auditorium/overlap.cuh:179-190). Here every transfer is a host-enqueued ncclSend/ncclRecv pair
// on a communication stream; arrival is ordered by CUDA events, so no kernel ever spins on a peer's flag, and
// received rows always land in this GPU's own memory before a GEMM tile loads them.
#include "ep_nccl.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "common.cuh"

namespace aristos {

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi& api() {
    static NcclApi a;
    static bool tried = false;
    if (tried) return a;
    tried = true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) return a;
#define LOAD(field, sym) \
    a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.handle, sym)); \
    if (!a.field) return a;
    LOAD(GetUniqueId, "ncclGetUniqueId")
    LOAD(CommInitRank, "ncclCommInitRank")
    LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(Send, "ncclSend")
    LOAD(Recv, "ncclRecv")
    LOAD(GroupStart, "ncclGroupStart")
    LOAD(GroupEnd, "ncclGroupEnd")
    LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    a.ok = true;
    return a;
}

aristos_status_t nccl_fail(ncclResult_t r, const char* what) {
    set_last_error("NCCL error %d (%s) in %s", (int)r, api().GetErrorString ? api().GetErrorString(r) : "?", what);
    return ARISTOS_ERR_NCCL;
}

#define NCCL_TRY(expr)                                         \
    do {                                                       \
        ncclResult_t _r = (expr);                              \
        if (_r != ncclSuccess) return nccl_fail(_r, #expr);    \
    } while (0)

}  // namespace

struct EpComm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};

aristos_status_t ep_unique_id(void* out) {
    if (!out) return ARISTOS_ERR_INVALID_ARG;
    if (!api().ok) { set_last_error("libnccl.so.2 could not be loaded"); return ARISTOS_ERR_NCCL; }
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
    ncclUniqueId id;
    NCCL_TRY(api().GetUniqueId(&id));
    memcpy(out, &id, sizeof(id));
    return ARISTOS_OK;
}

aristos_status_t ep_comm_create(const void* uid, int rank, int world, EpComm** out) {
    if (!uid || !out || world < 2 || rank < 0 || rank >= world) return ARISTOS_ERR_INVALID_ARG;
    if (!api().ok) { set_last_error("libnccl.so.2 could not be loaded"); return ARISTOS_ERR_NCCL; }
    ncclUniqueId id;
    memcpy(&id, uid, sizeof(id));
    EpComm* c = new EpComm();
    c->rank = rank;
    c->world = world;
    ncclResult_t r = api().CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) { delete c; return nccl_fail(r, "ncclCommInitRank"); }
    *out = c;
    return ARISTOS_OK;
}

void ep_comm_destroy(EpComm* c) {
    if (!c) return;
    if (c->comm && api().ok) api().CommDestroy(c->comm);
    delete c;
}

aristos_status_t ep_all_to_all_blocks(EpComm* c, const void* send_buf, void* recv_buf, int blocks_per_peer,
                                      size_t block_stride, size_t offset, size_t len, cudaStream_t stream) {
    if (!c || !send_buf || !recv_buf || blocks_per_peer <= 0) return ARISTOS_ERR_INVALID_ARG;
    if (len == 0) return ARISTOS_OK;
    const char* sb = static_cast<const char*>(send_buf);
    char* rb = static_cast<char*>(recv_buf);
    // own blocks: one strided device-to-device copy
    {
        const size_t base = (size_t)c->rank * blocks_per_peer * block_stride + offset;
        ARISTOS_CUDA_TRY(cudaMemcpy2DAsync(rb + base, block_stride, sb + base, block_stride, len, blocks_per_peer,
                                           cudaMemcpyDeviceToDevice, stream));
    }
    NCCL_TRY(api().GroupStart());
    for (int step = 1; step < c->world; ++step) {
        const int to = (c->rank + step) % c->world;
        const int from = (c->rank - step + c->world) % c->world;
        for (int b = 0; b < blocks_per_peer; ++b) {
            const size_t so = ((size_t)to * blocks_per_peer + b) * block_stride + offset;
            const size_t ro = ((size_t)from * blocks_per_peer + b) * block_stride + offset;
            ncclResult_t r = api().Send(sb + so, len, ncclInt8, to, c->comm, stream);
            if (r == ncclSuccess) r = api().Recv(rb + ro, len, ncclInt8, from, c->comm, stream);
            if (r != ncclSuccess) { api().GroupEnd(); return nccl_fail(r, "ncclSend/ncclRecv"); }
        }
    }
    NCCL_TRY(api().GroupEnd());
    return ARISTOS_OK;
}

}  // namespace aristos

extern "C" aristos_status_t aristos_nccl_unique_id(void* out_128_bytes) { return aristos::ep_unique_id(out_128_bytes); }
