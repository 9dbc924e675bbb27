// Expert-parallel exchange over peer memory (see ep_p2p.h).
//
// This is the B200 counterpart of the reference's device-initiated exchange (auditorium/overlap.cuh:94-153:
// nvshmemx_putmem_signal_nbi_block writes a tile into the peer's symmetric heap and raises a flag there, the consumer
// spins on nvshmem_signal_wait_until) and of its commented-out peer-store GEMM (mma.cuh:445-539): put = copy-engine
// write into the peer's IPC-mapped buffer, signal = epoch store into the peer's flag word, wait = stream memory
// operation on the local flag (no kernel spins, no SM is held while data is in flight).
#include "ep_p2p.h"

#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace aristos {

namespace {

constexpr size_t FLAG_BYTES = 4096;
constexpr int MAX_RANKS = 16;

struct FlagTargets {
    uint32_t* ptr[MAX_RANKS];
    int n;
};

// One warp: lane d stores the epoch into rank d's flag word for (kind, window, this rank).
__global__ void ep_signal_kernel(FlagTargets t, uint32_t epoch) {
    const int d = threadIdx.x;
    if (d < t.n) {
        __threadfence_system();
        *reinterpret_cast<volatile uint32_t*>(t.ptr[d]) = epoch;
        __threadfence_system();
    }
}

struct CountTargets {
    int32_t* ptr[MAX_RANKS];
};

// Row counts to their owners, then this rank's count flag at every rank (one CTA). With all.ptr[0] != nullptr every
// rank also gets the whole list (entry src_rank * E + e of its all-counts table).
__global__ void ep_counts_kernel(const int32_t* __restrict__ count, int E, int E_local, int src_rank, CountTargets dst,
                                 CountTargets all, FlagTargets t, uint32_t epoch) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int owner = e / E_local;
        const int c = count[e];
        dst.ptr[owner][src_rank * E_local + (e - owner * E_local)] = c;
        if (all.ptr[0] != nullptr)
            for (int d = 0; d < t.n; ++d) all.ptr[d][src_rank * E + e] = c;
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < t.n) {
        *reinterpret_cast<volatile uint32_t*>(t.ptr[threadIdx.x]) = epoch;
        __threadfence_system();
    }
}

typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

StreamWaitValue32Fn stream_wait_fn() {
    static StreamWaitValue32Fn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<StreamWaitValue32Fn>(sym);
    }
    return fn;
}

}  // namespace

struct EpP2P {
    int rank = 0, world = 1, groups = 0;
    size_t off_rcount = 0, off_allcount = 0, off_xr = 0, off_yg = 0, off_aux = 0, bytes = 0;
    char* local = nullptr;
    std::vector<char*> base;     // every rank's region as mapped into this process (own = local)
    uint32_t epoch = 0;
};

int ep_flag_word_index(int kind, int window, int src);
static size_t flag_index(const EpP2P*, int kind, int window, int src) {
    return (size_t)ep_flag_word_index(kind, window, src);
}

bool ep_transport_agreed(const int* ok_flags, int world) {
    for (int r = 0; r < world; ++r)
        if (!ok_flags[r]) return false;
    return world > 0;
}

// Every rank runs every collective step of the set-up, whatever happened to it locally: a rank whose allocation or
// mapping failed still takes part in both all-gathers and reports "not ok", and all ranks then take the same
// decision (peer memory only if it works everywhere). A rank that left early would leave the others in a collective.
aristos_status_t ep_p2p_create(EpComm* bootstrap, int rank, int world, int groups, size_t xr_bytes, size_t yg_bytes,
                               size_t aux_bytes, EpP2P** out) {
    if (!bootstrap || !out || world < 2 || world > MAX_RANKS) return ARISTOS_ERR_INVALID_ARG;
    static_assert(3 * EP_MAX_WINDOWS * MAX_RANKS * 4 <= FLAG_BYTES, "flag words fit their page");
    struct Hello {
        cudaIpcMemHandle_t handle;
        int ok;
        int pad[3];
    };
    EpP2P* p = new EpP2P();
    p->rank = rank;
    p->world = world;
    p->groups = groups;
    p->off_rcount = FLAG_BYTES;
    // the counts of every expert from every rank (world x E ints, E = groups): what dense packing of the received rows
    // needs at every sender before it gathers
    p->off_allcount = align_up(p->off_rcount + (size_t)groups * 4, 256);
    p->off_xr = align_up(p->off_allcount + (size_t)world * groups * 4, 1024);
    p->off_yg = align_up(p->off_xr + xr_bytes, 1024);
    p->off_aux = align_up(p->off_yg + yg_bytes, 1024);
    p->bytes = align_up(p->off_aux + aux_bytes, 1024);
    p->base.assign(world, nullptr);
    char local_error[256] = "";
    Hello mine;
    memset(&mine, 0, sizeof(mine));
    // ---- local part: may fail without leaving the protocol
    int ok = stream_wait_fn() != nullptr;
    if (!ok) snprintf(local_error, sizeof(local_error), "cuStreamWaitValue32 is not available from the driver");
    // host-injected failure for the tests of the agreement (nothing on the GPU fails)
    const char* inject = getenv("ARISTOS_EP_INJECT_P2P_FAIL");
    const int inject_rank = inject ? atoi(inject) : -1;
    const bool inject_alloc = inject_rank == rank && getenv("ARISTOS_EP_INJECT_STAGE") &&
                              !strcmp(getenv("ARISTOS_EP_INJECT_STAGE"), "alloc");
    if (ok) {
        cudaError_t e = inject_alloc ? cudaErrorMemoryAllocation : cudaMalloc(reinterpret_cast<void**>(&p->local), p->bytes);
        if (e == cudaSuccess) e = cudaMemset(p->local, 0, p->off_xr);
        if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine.handle, p->local);
        if (e != cudaSuccess) {
            ok = 0;
            snprintf(local_error, sizeof(local_error), "exchange region of %zu bytes: %s", p->bytes, cudaGetErrorString(e));
            cudaGetLastError();
        }
    }
    mine.ok = ok;
    p->base[rank] = p->local;
    // ---- collective part 1: handles and "allocated" flags (also the barrier that orders every rank's flag clearing
    // before any peer's first store)
    Hello* d_all = nullptr;
    std::vector<Hello> all(world);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&d_all), sizeof(Hello) * (world + 1));
    if (e != cudaSuccess) { ep_p2p_destroy(p); return cuda_fail(e, "peer-memory exchange set-up (staging)"); }
    aristos_status_t st = ARISTOS_OK;
    e = cudaMemcpy(d_all + world, &mine, sizeof(mine), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) st = ep_allgather_bytes(bootstrap, d_all + world, d_all, sizeof(Hello), nullptr);
    if (e == cudaSuccess && st == ARISTOS_OK) e = cudaStreamSynchronize(nullptr);
    if (e == cudaSuccess && st == ARISTOS_OK) e = cudaMemcpy(all.data(), d_all, sizeof(Hello) * world, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || st != ARISTOS_OK) {
        cudaFree(d_all);
        ep_p2p_destroy(p);
        return st != ARISTOS_OK ? st : cuda_fail(e, "peer-memory exchange set-up (handle all-gather)");
    }
    std::vector<int> flags(world);
    for (int r = 0; r < world; ++r) flags[r] = all[r].ok;
    int mapped_ok = ep_transport_agreed(flags.data(), world) ? 1 : 0;
    // ---- local part 2: map the peers' regions (only when every rank has one)
    if (mapped_ok) {
        for (int r = 0; r < world && mapped_ok; ++r) {
            if (r == rank) continue;
            void* mapped = nullptr;
            cudaError_t me = (inject_rank == rank && !inject_alloc) ? cudaErrorInvalidResourceHandle
                                 : cudaIpcOpenMemHandle(&mapped, all[r].handle, cudaIpcMemLazyEnablePeerAccess);
            if (me != cudaSuccess) {
                mapped_ok = 0;
                snprintf(local_error, sizeof(local_error), "mapping rank %d's exchange region: %s", r, cudaGetErrorString(me));
                cudaGetLastError();
            }
            p->base[r] = static_cast<char*>(mapped);
        }
    }
    // ---- collective part 2: did every rank map every peer?
    mine.ok = mapped_ok;
    e = cudaMemcpy(d_all + world, &mine, sizeof(mine), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) st = ep_allgather_bytes(bootstrap, d_all + world, d_all, sizeof(Hello), nullptr);
    if (e == cudaSuccess && st == ARISTOS_OK) e = cudaStreamSynchronize(nullptr);
    if (e == cudaSuccess && st == ARISTOS_OK) e = cudaMemcpy(all.data(), d_all, sizeof(Hello) * world, cudaMemcpyDeviceToHost);
    cudaFree(d_all);
    if (e != cudaSuccess || st != ARISTOS_OK) {
        ep_p2p_destroy(p);
        return st != ARISTOS_OK ? st : cuda_fail(e, "peer-memory exchange set-up (agreement all-gather)");
    }
    for (int r = 0; r < world; ++r) flags[r] = all[r].ok;
    if (!ep_transport_agreed(flags.data(), world)) {
        int first_bad = 0;
        while (first_bad < world && flags[first_bad]) ++first_bad;
        ep_p2p_destroy(p);
        if (local_error[0]) set_last_error("peer-memory transport unavailable on this rank: %s", local_error);
        else set_last_error("peer-memory transport unavailable on rank %d; every rank falls back together", first_bad);
        return ARISTOS_ERR_UNSUPPORTED;
    }
    *out = p;
    return ARISTOS_OK;
}

void ep_p2p_destroy(EpP2P* p) {
    if (!p) return;
    for (int r = 0; r < p->world; ++r)
        if (r != p->rank && p->base[r]) cudaIpcCloseMemHandle(p->base[r]);
    if (p->local) cudaFree(p->local);
    delete p;
}

void* ep_p2p_xr(EpP2P* p) { return p->local + p->off_xr; }
void* ep_p2p_yg(EpP2P* p) { return p->local + p->off_yg; }
void* ep_p2p_aux(EpP2P* p) { return p->local + p->off_aux; }

void ep_p2p_peer_ptrs(EpP2P* p, int which, void** out) {
    const size_t off = which == EP_BUF_XR ? p->off_xr
                       : (which == EP_BUF_YG ? p->off_yg : (which == EP_BUF_RCOUNT ? p->off_rcount : p->off_aux));
    for (int r = 0; r < p->world; ++r) out[r] = p->base[r] + off;
}
int32_t* ep_p2p_rcount(EpP2P* p) { return reinterpret_cast<int32_t*>(p->local + p->off_rcount); }
int32_t* ep_p2p_allcount(EpP2P* p) { return reinterpret_cast<int32_t*>(p->local + p->off_allcount); }
uint32_t ep_p2p_begin(EpP2P* p) { return ++p->epoch; }

aristos_status_t ep_p2p_push(EpP2P* p, int which, const void* send_buf, int blocks_per_peer, size_t block_stride,
                             size_t offset, size_t len, cudaStream_t stream) {
    if (!p || !send_buf || blocks_per_peer <= 0) return ARISTOS_ERR_INVALID_ARG;
    if (len == 0) return ARISTOS_OK;
    const size_t dst_off = which == EP_FLAG_IN ? p->off_xr : (which == EP_FLAG_RET ? p->off_yg : p->off_rcount);
    const char* sb = static_cast<const char*>(send_buf);
    for (int step = 0; step < p->world; ++step) {
        const int d = (p->rank + step) % p->world;      // own blocks first, then the peers in ring order
        const char* src = sb + (size_t)d * blocks_per_peer * block_stride + offset;
        char* dst = p->base[d] + dst_off + (size_t)p->rank * blocks_per_peer * block_stride + offset;
        ARISTOS_CUDA_TRY(cudaMemcpy2DAsync(dst, block_stride, src, block_stride, len, blocks_per_peer,
                                           cudaMemcpyDeviceToDevice, stream));
    }
    return ARISTOS_OK;
}

aristos_status_t ep_p2p_signal(EpP2P* p, int kind, int window, cudaStream_t stream) {
    if (!p || window < 0 || window >= EP_MAX_WINDOWS) return ARISTOS_ERR_INVALID_ARG;
    FlagTargets t;
    t.n = p->world;
    for (int d = 0; d < p->world; ++d)
        t.ptr[d] = reinterpret_cast<uint32_t*>(p->base[d]) + flag_index(p, kind, window, p->rank);
    ep_signal_kernel<<<1, 32, 0, stream>>>(t, p->epoch);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

aristos_status_t ep_p2p_wait(EpP2P* p, int kind, int window, cudaStream_t stream) {
    if (!p || window < 0 || window >= EP_MAX_WINDOWS) return ARISTOS_ERR_INVALID_ARG;
    StreamWaitValue32Fn wait = stream_wait_fn();
    for (int src = 0; src < p->world; ++src) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(p->local) + flag_index(p, kind, window, src);
        const CUresult r = wait(reinterpret_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), p->epoch,
                                CU_STREAM_WAIT_VALUE_GEQ);
        if (r != CUDA_SUCCESS) { set_last_error("cuStreamWaitValue32 failed with %d", (int)r); return ARISTOS_ERR_CUDA; }
    }
    return ARISTOS_OK;
}

const uint32_t* ep_p2p_flags(const EpP2P* p, int kind, int window) {
    return reinterpret_cast<const uint32_t*>(p->local) + flag_index(p, kind, window, 0);
}
uint32_t ep_p2p_epoch(const EpP2P* p) { return p->epoch; }

aristos_status_t ep_p2p_send_counts(EpP2P* p, const int32_t* count, int E, int E_local, cudaStream_t stream,
                                    bool to_all) {
    if (!p || !count || E_local <= 0 || E != E_local * p->world || E != p->groups) return ARISTOS_ERR_INVALID_ARG;
    FlagTargets t;
    CountTargets c, all;
    t.n = p->world;
    for (int d = 0; d < MAX_RANKS; ++d) all.ptr[d] = nullptr;
    for (int d = 0; d < p->world; ++d) {
        t.ptr[d] = reinterpret_cast<uint32_t*>(p->base[d]) + flag_index(p, EP_FLAG_COUNT, 0, p->rank);
        c.ptr[d] = reinterpret_cast<int32_t*>(p->base[d] + p->off_rcount);
        if (to_all) all.ptr[d] = reinterpret_cast<int32_t*>(p->base[d] + p->off_allcount);
    }
    ep_counts_kernel<<<1, 256, 0, stream>>>(count, E, E_local, p->rank, c, all, t, p->epoch);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

// ---- the flag protocol as host-side functions (the device-side stores and waits follow the same layout and the same
// cyclic comparison; exported for tests that run the protocol among CPU ranks) ------------------------------------
int ep_flag_words() { return 3 * EP_MAX_WINDOWS * MAX_RANKS; }
int ep_flag_word_index(int kind, int window, int src) {
    if (kind < 0 || kind > 2 || window < 0 || window >= EP_MAX_WINDOWS || src < 0 || src >= MAX_RANKS) return -1;
    return (kind * EP_MAX_WINDOWS + window) * MAX_RANKS + src;
}
// Bit s set: source rank s has not yet raised its (kind, window) flag to `epoch` (cyclic comparison: a flag that is
// ahead of the epoch counts as arrived).
uint32_t ep_flags_pending(const uint32_t* words, uint32_t epoch, int world, int kind, int window) {
    uint32_t pending = 0;
    for (int s = 0; s < world && s < MAX_RANKS; ++s)
        if (static_cast<int32_t>(words[ep_flag_word_index(kind, window, s)] - epoch) < 0) pending |= 1u << s;
    return pending;
}
// Release: every flag word of this rank takes the current epoch, so nothing of the current forward is pending.
void ep_flags_release(uint32_t* words, uint32_t epoch) {
    for (int i = 0; i < ep_flag_words(); ++i)
        if (static_cast<int32_t>(words[i] - epoch) < 0) words[i] = epoch;
}

aristos_status_t ep_p2p_release_local_waits(EpP2P* p) {
    if (!p) return ARISTOS_ERR_INVALID_ARG;
    // copies on the legacy stream would queue behind the stalled streams: use a non-blocking stream of its own.
    // Peers cannot be ahead of this rank's epoch (they need its flags to get there), so raising the lagging words
    // to the epoch never undoes a store of theirs.
    std::vector<uint32_t> words(ep_flag_words(), 0u);
    cudaStream_t s = nullptr;
    ARISTOS_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    cudaError_t e = cudaMemcpyAsync(words.data(), p->local, words.size() * 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess) {
        ep_flags_release(words.data(), p->epoch);
        e = cudaMemcpyAsync(p->local, words.data(), words.size() * 4, cudaMemcpyHostToDevice, s);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaStreamDestroy(s);
    if (e != cudaSuccess) return cuda_fail(e, "release of the local exchange flags");
    return ARISTOS_OK;
}

}  // namespace aristos

extern "C" int aristos_ep_transport_agreed(const int* ok_flags, int world) {
    if (!ok_flags || world < 1) return 0;
    return aristos::ep_transport_agreed(ok_flags, world) ? 1 : 0;
}

extern "C" int aristos_ep_flag_words(void) { return aristos::ep_flag_words(); }
extern "C" int aristos_ep_flag_word_index(int kind, int window, int src) {
    return aristos::ep_flag_word_index(kind, window, src);
}
extern "C" uint32_t aristos_ep_flags_pending(const uint32_t* words, uint32_t epoch, int world, int kind, int window) {
    if (!words || world < 1 || aristos::ep_flag_word_index(kind, window, 0) < 0) return 0xffffffffu;
    return aristos::ep_flags_pending(words, epoch, world, kind, window);
}
extern "C" void aristos_ep_flags_release(uint32_t* words, uint32_t epoch) {
    if (words) aristos::ep_flags_release(words, epoch);
}
