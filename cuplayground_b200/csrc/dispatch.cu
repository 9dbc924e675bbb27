// Dispatch: capacity-bounded per-expert token lists, overflow dropped in token order, and the gather of token
// rows into expert-major order.
//
// The reference has no dispatch; the nearest code is the task-queue bookkeeping of its in-kernel schedulers
// (auditorium/scheduling.cuh:218-252 builds per-producer queue heads and a ready queue). The contract here:
// walking the (token, j) assignments in token-major order, the position of an assignment inside expert e is the
// number of earlier assignments to e; it is kept iff position < capacity. Three integer kernels make that walk
// parallel without depending on the order in which atomics land:
//   1. count : every CTA owns a contiguous chunk of assignments and histograms it (warp-aggregated shared atomics)
//   2. scan  : exclusive prefix over chunks per expert -> chunk bases, count[e] = min(total, capacity)
//   3. assign: every warp owns a contiguous sub-chunk; per-warp histograms + an in-CTA prefix give each warp its
//              base, __match_any_sync groups lanes that picked the same expert and the lane's rank inside its
//              group is its offset, so positions follow token order exactly.
#include <atomic>
#include "common.cuh"

namespace aristos {

constexpr int DSP_THREADS = 256;
constexpr int DSP_WARPS = DSP_THREADS / 32;
constexpr int DSP_STEPS = 8;                             // 32-assignment steps per warp
constexpr int DSP_CHUNK = DSP_WARPS * DSP_STEPS * 32;    // assignments per CTA (2048)

__global__ void __launch_bounds__(DSP_THREADS)
dispatch_count_kernel(const int32_t* __restrict__ topk_idx, int n_assign, int E, int32_t* __restrict__ chunk_hist,
                      int32_t* __restrict__ dev_status) {
    extern __shared__ int32_t s_hist[];  // [E]
    for (int e = threadIdx.x; e < E; e += DSP_THREADS) s_hist[e] = 0;
    __syncthreads();
    const int base = blockIdx.x * DSP_CHUNK;
    for (int off = threadIdx.x; off < DSP_CHUNK; off += DSP_THREADS) {
        const int i = base + off;
        int e = (i < n_assign) ? topk_idx[i] : -1;
        if (i < n_assign && (e < 0 || e >= E)) {
            if (dev_status) atomicOr(dev_status, DEV_FAULT_BOUNDS);
            e = -1;
        }
        const unsigned mask = __match_any_sync(0xffffffffu, e);
        const int leader = __ffs(mask) - 1;
        if (e >= 0 && (threadIdx.x & 31) == leader) atomicAdd(&s_hist[e], __popc(mask));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += DSP_THREADS) chunk_hist[(size_t)blockIdx.x * E + e] = s_hist[e];
}

__global__ void dispatch_scan_kernel(int32_t* __restrict__ chunk_hist, int nchunks, int E, int cap,
                                     int32_t* __restrict__ count) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    int running = 0;
    for (int c = 0; c < nchunks; ++c) {
        const int v = chunk_hist[(size_t)c * E + e];
        chunk_hist[(size_t)c * E + e] = running;
        running += v;
    }
    count[e] = min(running, cap);
}

__global__ void __launch_bounds__(DSP_THREADS)
dispatch_assign_kernel(const int32_t* __restrict__ topk_idx, int n_assign, int k, int E, int cap,
                       const int32_t* __restrict__ chunk_base, int32_t* __restrict__ slot_of,
                       int32_t* __restrict__ token_of_slot) {
    extern __shared__ int32_t s_warp_hist[];  // [DSP_WARPS][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < DSP_WARPS * E; i += DSP_THREADS) s_warp_hist[i] = 0;
    __syncthreads();
    int32_t* my_hist = s_warp_hist + warp * E;
    const int base = blockIdx.x * DSP_CHUNK + warp * (DSP_STEPS * 32);
    int e_step[DSP_STEPS];
#pragma unroll
    for (int s = 0; s < DSP_STEPS; ++s) {
        const int i = base + s * 32 + lane;
        int e = (i < n_assign) ? topk_idx[i] : -1;
        if (e < 0 || e >= E) e = -1;
        e_step[s] = e;
        const unsigned mask = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == __ffs(mask) - 1) my_hist[e] += __popc(mask);
        __syncwarp();
    }
    __syncthreads();
    // exclusive prefix over the warps of this CTA, seeded with the chunk's global base
    for (int e = threadIdx.x; e < E; e += DSP_THREADS) {
        int running = chunk_base[(size_t)blockIdx.x * E + e];
        for (int w = 0; w < DSP_WARPS; ++w) {
            const int v = s_warp_hist[w * E + e];
            s_warp_hist[w * E + e] = running;
            running += v;
        }
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < DSP_STEPS; ++s) {
        const int i = base + s * 32 + lane;
        const int e = e_step[s];
        const unsigned mask = __match_any_sync(0xffffffffu, e);
        int pos = 0;
        if (e >= 0) pos = my_hist[e] + __popc(mask & ((1u << lane) - 1u));
        __syncwarp();
        if (e >= 0 && lane == __ffs(mask) - 1) my_hist[e] += __popc(mask);
        __syncwarp();
        if (i < n_assign) {
            int slot = -1;
            if (e >= 0 && pos < cap) {
                slot = e * cap + pos;
                token_of_slot[slot] = i / k;
            }
            slot_of[i] = slot;
        }
    }
}

// xg[slot_of[t,j]] = x[t]; one warp per token, each row read once and written up to k times.
template <int MAXK>
__global__ void __launch_bounds__(256)
permute_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ slot_of, int S, int k, int row_vec,
                    uint4* __restrict__ xg) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= S) return;
    int slots[MAXK];
#pragma unroll
    for (int j = 0; j < MAXK; ++j) slots[j] = (j < k) ? slot_of[(size_t)warp * k + j] : -1;
    const uint4* src = x + (size_t)warp * row_vec;
    for (int c0 = 0; c0 < row_vec; c0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * 32 + lane;
            if (c < row_vec) v[u] = __ldg(src + c);
        }
#pragma unroll
        for (int j = 0; j < MAXK; ++j) {
            if (slots[j] < 0) continue;
            uint4* dst = xg + (size_t)slots[j] * row_vec;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < row_vec) dst[c] = v[u];
            }
        }
    }
}

}  // namespace aristos

using namespace aristos;

extern "C" size_t aristos_dispatch_scratch_bytes(int S, int k, int E) {
    if (S < 0 || k <= 0 || E <= 0) return 0;
    const int64_t n = (int64_t)S * k;
    const int64_t nchunks = (n + DSP_CHUNK - 1) / DSP_CHUNK;
    return align_up((size_t)(nchunks > 0 ? nchunks : 1) * (size_t)E * sizeof(int32_t), 256);
}

namespace aristos {
// Internal form with a device status word (the public entry passes NULL).
aristos_status_t dispatch_impl(const int32_t* topk_idx, int S, int k, int E, int cap, int32_t* count,
                               int32_t* slot_of, int32_t* token_of_slot, void* scratch, size_t scratch_bytes,
                               int32_t* dev_status, cudaStream_t st) {
    if ((!topk_idx && S > 0) || (!slot_of && S > 0) || !count || !token_of_slot || !scratch) {
        set_last_error("dispatch: NULL pointer");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (S < 0 || k <= 0 || E <= 0 || cap <= 0 || E > 1024) { set_last_error("dispatch: bad size"); return ARISTOS_ERR_INVALID_ARG; }
    if ((int64_t)E * cap > 0x7fffffffLL || (int64_t)S * k > 0x7fffffffLL) { set_last_error("dispatch: E*cap or S*k overflows int32"); return ARISTOS_ERR_CONFIG; }
    if (scratch_bytes < aristos_dispatch_scratch_bytes(S, k, E)) { set_last_error("dispatch: scratch too small"); return ARISTOS_ERR_WORKSPACE; }
    const int n = S * k;
    const int nchunks = ceil_div(n, DSP_CHUNK);
    int32_t* chunk_hist = static_cast<int32_t*>(scratch);
    ARISTOS_CUDA_TRY(cudaMemsetAsync(token_of_slot, 0xFF, sizeof(int32_t) * (size_t)E * cap, st));
    if (n == 0) {
        ARISTOS_CUDA_TRY(cudaMemsetAsync(count, 0, sizeof(int32_t) * (size_t)E, st));
        return ARISTOS_OK;
    }
    dispatch_count_kernel<<<nchunks, DSP_THREADS, sizeof(int32_t) * E, st>>>(topk_idx, n, E, chunk_hist, dev_status);
    ARISTOS_COUNT_LAUNCH();
    dispatch_scan_kernel<<<ceil_div(E, 128), 128, 0, st>>>(chunk_hist, nchunks, E, cap, count);
    ARISTOS_COUNT_LAUNCH();
    dispatch_assign_kernel<<<nchunks, DSP_THREADS, sizeof(int32_t) * DSP_WARPS * E, st>>>(
        topk_idx, n, k, E, cap, chunk_hist, slot_of, token_of_slot);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}
}  // namespace aristos

extern "C" aristos_status_t aristos_dispatch(const int32_t* topk_idx, int S, int k, int E, int cap, int32_t* count,
                                             int32_t* slot_of, int32_t* token_of_slot, void* scratch,
                                             size_t scratch_bytes, void* stream) {
    return dispatch_impl(topk_idx, S, k, E, cap, count, slot_of, token_of_slot, scratch, scratch_bytes, nullptr,
                         static_cast<cudaStream_t>(stream));
}

// ---- dispatch without any allocation ---------------------------------------------------------------------------------
// The per-chunk histograms of the dispatch live in this fixed array instead of caller-provided scratch memory. Every
// GPU that loads the library holds these 64 KiB until the process exits.
constexpr int STATIC_MAX_ASSIGN = 131072;                              // S * k
constexpr int STATIC_MAX_EXPERTS = 256;
constexpr int STATIC_MAX_CHUNKS = STATIC_MAX_ASSIGN / aristos::DSP_CHUNK;
static __device__ __align__(256) int32_t g_dispatch_static_scratch[STATIC_MAX_CHUNKS * STATIC_MAX_EXPERTS];

extern "C" aristos_status_t aristos_dispatch_static(const int32_t* topk_idx, int S, int k, int E, int cap,
                                                    int32_t* count, int32_t* slot_of, int32_t* token_of_slot,
                                                    void* stream) {
    if (S < 0 || k <= 0 || E <= 0) { set_last_error("dispatch_static: bad size"); return ARISTOS_ERR_INVALID_ARG; }
    if ((int64_t)S * k > STATIC_MAX_ASSIGN || E > STATIC_MAX_EXPERTS) {
        set_last_error("dispatch_static: S*k = %lld (limit %d) or E = %d (limit %d) exceeds the built-in scratch; "
                       "use aristos_dispatch with caller scratch", (long long)S * k, STATIC_MAX_ASSIGN, E,
                       STATIC_MAX_EXPERTS);
        return ARISTOS_ERR_CONFIG;
    }
    // The array's name is only a host-side handle: the kernels need its device address, looked up once per device
    // with that device current.
    // Two host threads that make the first call on one device at the same time both look the address up and store the
    // same value; the atomic makes that store and the later loads well defined.
    constexpr int MAX_DEVICES = 64;
    static std::atomic<int32_t*> scratch_of_device[MAX_DEVICES];
    int dev = 0;
    ARISTOS_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) { set_last_error("dispatch_static: device index %d not supported", dev); return ARISTOS_ERR_UNSUPPORTED; }
    int32_t* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
    if (!scratch) {
        void* p = nullptr;
        ARISTOS_CUDA_TRY(cudaGetSymbolAddress(&p, g_dispatch_static_scratch));
        scratch = static_cast<int32_t*>(p);
        scratch_of_device[dev].store(scratch, std::memory_order_release);
    }
    return dispatch_impl(topk_idx, S, k, E, cap, count, slot_of, token_of_slot, scratch,
                         sizeof(int32_t) * STATIC_MAX_CHUNKS * STATIC_MAX_EXPERTS, nullptr,
                         static_cast<cudaStream_t>(stream));
}

extern "C" aristos_status_t aristos_permute(const void* x, const int32_t* slot_of, int S, int k, int H, int dtype,
                                            void* xg, void* stream) {
    if (!x || !slot_of || !xg) { set_last_error("permute: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    const size_t eb = dtype_bytes(dtype);
    if (eb == 0 || S < 0 || k <= 0 || k > 16 || H <= 0 || ((size_t)H * eb) % 16 != 0) {
        set_last_error("permute: bad size (row bytes must be a multiple of 16, k <= 16)");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (!aligned16(x) || !aligned16(xg)) { set_last_error("permute: pointers must be 16-byte aligned"); return ARISTOS_ERR_INVALID_ARG; }
    if (S == 0) return ARISTOS_OK;
    const int row_vec = (int)((size_t)H * eb / 16);
    const int grid = ceil_div(S, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (k <= 2) permute_rows_kernel<2><<<grid, 256, 0, st>>>((const uint4*)x, slot_of, S, k, row_vec, (uint4*)xg);
    else if (k <= 4) permute_rows_kernel<4><<<grid, 256, 0, st>>>((const uint4*)x, slot_of, S, k, row_vec, (uint4*)xg);
    else if (k <= 8) permute_rows_kernel<8><<<grid, 256, 0, st>>>((const uint4*)x, slot_of, S, k, row_vec, (uint4*)xg);
    else permute_rows_kernel<16><<<grid, 256, 0, st>>>((const uint4*)x, slot_of, S, k, row_vec, (uint4*)xg);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}
