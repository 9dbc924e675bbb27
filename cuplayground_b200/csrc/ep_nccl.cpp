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
#include <vector>

#include "common.cuh"

namespace aristos {

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;   // optional
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
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
    LOAD(AllGather, "ncclAllGather")
    LOAD(GroupStart, "ncclGroupStart")
    LOAD(GroupEnd, "ncclGroupEnd")
    LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    a.CommInitRankConfig = reinterpret_cast<decltype(a.CommInitRankConfig)>(dlsym(a.handle, "ncclCommInitRankConfig"));
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

aristos_status_t ep_comm_create(const void* uid, int rank, int world, int max_ctas, EpComm** out) {
    if (!uid || !out || world < 2 || rank < 0 || rank >= world) return ARISTOS_ERR_INVALID_ARG;
    if (!api().ok) { set_last_error("libnccl.so.2 could not be loaded"); return ARISTOS_ERR_NCCL; }
    ncclUniqueId id;
    memcpy(&id, uid, sizeof(id));
    EpComm* c = new EpComm();
    c->rank = rank;
    c->world = world;
    ncclResult_t r;
    if (max_ctas > 0 && api().CommInitRankConfig) {
        // bound the CTAs of NCCL's copy kernels: they run beside the persistent GEMM grid, which leaves them that
        // many SMs
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.maxCTAs = max_ctas;
        config.minCTAs = 1;
        r = api().CommInitRankConfig(&c->comm, world, id, rank, &config);
    } else {
        r = api().CommInitRank(&c->comm, world, id, rank);
    }
    if (r != ncclSuccess) { delete c; return nccl_fail(r, "ncclCommInitRank"); }
    *out = c;
    return ARISTOS_OK;
}

void ep_comm_destroy(EpComm* c) {
    if (!c) return;
    if (c->comm && api().ok) api().CommDestroy(c->comm);
    delete c;
}

aristos_status_t ep_allgather_bytes(EpComm* c, const void* send_dev, void* recv_dev, size_t bytes_per_rank,
                                    cudaStream_t stream) {
    if (!c || !send_dev || !recv_dev) return ARISTOS_ERR_INVALID_ARG;
    NCCL_TRY(api().AllGather(send_dev, recv_dev, bytes_per_rank, ncclInt8, c->comm, stream));
    return ARISTOS_OK;
}

// The exchange of one row window as a flat list of transfers; entry 0 is the rank's own copy.
std::vector<EpTransfer> ep_exchange_plan(int rank, int world, int blocks_per_peer, size_t block_stride, size_t offset,
                                         size_t len) {
    std::vector<EpTransfer> plan;
    for (int step = 0; step < world; ++step) {
        const int to = (rank + step) % world;
        const int from = (rank - step + world) % world;
        for (int b = 0; b < blocks_per_peer; ++b) {
            EpTransfer t;
            t.send_to = to;
            t.recv_from = from;
            t.send_offset = ((size_t)to * blocks_per_peer + b) * block_stride + offset;
            t.recv_offset = ((size_t)from * blocks_per_peer + b) * block_stride + offset;
            t.bytes = len;
            plan.push_back(t);
        }
    }
    return plan;
}

void ep_row_windows(int cap, int max_windows, int min_rows, int* window_rows, int* windows) {
    int n = max_windows < 1 ? 1 : max_windows;
    while (n > 1 && (cap + n - 1) / n < min_rows) --n;
    const int rows = ((cap + n - 1) / n + 127) / 128 * 128;
    *window_rows = rows;
    *windows = (cap + rows - 1) / rows;
}

aristos_status_t ep_all_to_all_blocks(EpComm* c, const void* send_buf, void* recv_buf, int blocks_per_peer,
                                      size_t block_stride, size_t offset, size_t len, cudaStream_t stream) {
    if (!c || !send_buf || !recv_buf || blocks_per_peer <= 0) return ARISTOS_ERR_INVALID_ARG;
    if (len == 0) return ARISTOS_OK;
    const char* sb = static_cast<const char*>(send_buf);
    char* rb = static_cast<char*>(recv_buf);
    const std::vector<EpTransfer> plan = ep_exchange_plan(c->rank, c->world, blocks_per_peer, block_stride, offset, len);
    // own blocks (the first blocks_per_peer entries): one strided device-to-device copy
    ARISTOS_CUDA_TRY(cudaMemcpy2DAsync(rb + plan[0].recv_offset, block_stride, sb + plan[0].send_offset, block_stride,
                                       len, blocks_per_peer, cudaMemcpyDeviceToDevice, stream));
    NCCL_TRY(api().GroupStart());
    for (size_t i = blocks_per_peer; i < plan.size(); ++i) {
        const EpTransfer& t = plan[i];
        ncclResult_t r = api().Send(sb + t.send_offset, t.bytes, ncclInt8, t.send_to, c->comm, stream);
        if (r == ncclSuccess) r = api().Recv(rb + t.recv_offset, t.bytes, ncclInt8, t.recv_from, c->comm, stream);
        if (r != ncclSuccess) { api().GroupEnd(); return nccl_fail(r, "ncclSend/ncclRecv"); }
    }
    NCCL_TRY(api().GroupEnd());
    return ARISTOS_OK;
}

}  // namespace aristos

extern "C" aristos_status_t aristos_nccl_unique_id(void* out_128_bytes) { return aristos::ep_unique_id(out_128_bytes); }

extern "C" int aristos_ep_exchange_plan(int rank, int world, int blocks_per_peer, size_t block_stride, size_t offset,
                                        size_t len, int64_t* out, int max_entries) {
    if (world < 1 || rank < 0 || rank >= world || blocks_per_peer < 1) return -1;
    const std::vector<aristos::EpTransfer> plan =
        aristos::ep_exchange_plan(rank, world, blocks_per_peer, block_stride, offset, len);
    if (out) {
        for (size_t i = 0; i < plan.size() && (int)i < max_entries; ++i) {
            out[5 * i + 0] = plan[i].send_to;
            out[5 * i + 1] = (int64_t)plan[i].send_offset;
            out[5 * i + 2] = plan[i].recv_from;
            out[5 * i + 3] = (int64_t)plan[i].recv_offset;
            out[5 * i + 4] = (int64_t)plan[i].bytes;
        }
    }
    return (int)plan.size();
}

extern "C" aristos_status_t aristos_ep_row_windows(int cap, int* window_rows, int* windows) {
    if (cap < 1 || !window_rows || !windows) return ARISTOS_ERR_INVALID_ARG;
    aristos::ep_row_windows(cap, 4, 512, window_rows, windows);
    return ARISTOS_OK;
}
