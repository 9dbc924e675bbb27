// aristos_expert_ffn: argument checks and the per-dtype kernels behind the C ABI.
#include "common.cuh"
#include "ffn_internal.h"
#include "ptx_sm100.cuh"

using namespace aristos;

extern "C" aristos_status_t aristos_expert_ffn_fp8(const void* xq, const float* sx, const int32_t* count, int groups,
                                                   int rows_per_group, int experts, const void* w1q, const float* s1,
                                                   const void* w3q, const float* s3, const void* w2q, const float* s2,
                                                   void* h_scratch, void* hq_scratch, float* sh_scratch, void* y,
                                                   int H, int I, int hidden_act, int row_begin, int row_end,
                                                   int sm_limit, int32_t* dev_status, void* stream) {
    if (!xq || !sx || !count || !w1q || !s1 || !w2q || !s2 || !h_scratch || !hq_scratch || !sh_scratch || !y) {
        set_last_error("expert_ffn_fp8: NULL pointer");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (hidden_act == ARISTOS_ACT_SWIGLU && (!w3q || !s3)) { set_last_error("expert_ffn_fp8: SwiGLU needs w3 and its scales"); return ARISTOS_ERR_INVALID_ARG; }
    if (hidden_act < 0 || hidden_act > 2) { set_last_error("expert_ffn_fp8: hidden_act must be 0, 1 or 2"); return ARISTOS_ERR_INVALID_ARG; }
    if (groups < 0 || rows_per_group <= 0 || experts <= 0 || H <= 0 || I <= 0 || row_begin < 0 || row_end < row_begin ||
        row_end > rows_per_group) {
        set_last_error("expert_ffn_fp8: bad size");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (!aligned16(xq) || !aligned16(w1q) || !aligned16(w2q) || !aligned16(h_scratch) || !aligned16(hq_scratch) ||
        !aligned16(y) || (w3q && !aligned16(w3q))) {
        set_last_error("expert_ffn_fp8: pointers must be 16-byte aligned");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (groups == 0 || row_end == row_begin) return ARISTOS_OK;
    return expert_ffn_fp8_sm100(xq, sx, count, groups, rows_per_group, experts, w1q, s1, w3q, s3, w2q, s2, h_scratch,
                                hq_scratch, sh_scratch, y, H, I, hidden_act, row_begin, row_end, sm_limit, dev_status,
                                static_cast<cudaStream_t>(stream));
}

extern "C" aristos_status_t aristos_expert_ffn(const void* xg, const int32_t* count, int groups, int rows_per_group,
                                               int experts, const void* w1, const void* w3, const void* w2,
                                               void* h_scratch, void* y, int H, int I, int hidden_act, int dtype,
                                               int row_begin, int row_end, int sm_limit, int32_t* dev_status,
                                               void* stream) {
    return aristos_expert_ffn_bias(xg, count, groups, rows_per_group, experts, w1, w3, w2, nullptr, nullptr, nullptr,
                                   h_scratch, y, H, I, hidden_act, dtype, row_begin, row_end, sm_limit, dev_status,
                                   stream);
}

extern "C" aristos_status_t aristos_expert_ffn_bias(const void* xg, const int32_t* count, int groups,
                                                    int rows_per_group, int experts, const void* w1, const void* w3,
                                                    const void* w2, const void* b1, const void* b3, const void* b2,
                                                    void* h_scratch, void* y, int H, int I, int hidden_act, int dtype,
                                                    int row_begin, int row_end, int sm_limit, int32_t* dev_status,
                                                    void* stream) {
    if (!xg || !count || !w1 || !w2 || !h_scratch || !y) { set_last_error("expert_ffn: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (hidden_act == ARISTOS_ACT_SWIGLU && !w3) { set_last_error("expert_ffn: SwiGLU needs w3"); return ARISTOS_ERR_INVALID_ARG; }
    if (hidden_act < 0 || hidden_act > 2) { set_last_error("expert_ffn: hidden_act must be 0, 1 or 2"); return ARISTOS_ERR_INVALID_ARG; }
    if (groups < 0 || rows_per_group <= 0 || experts <= 0 || H <= 0 || I <= 0 || row_begin < 0 || row_end < row_begin ||
        row_end > rows_per_group) {
        set_last_error("expert_ffn: bad size");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (!aligned16(xg) || !aligned16(w1) || !aligned16(w2) || !aligned16(h_scratch) || !aligned16(y) ||
        (w3 && !aligned16(w3)) || (b1 && !aligned16(b1)) || (b3 && !aligned16(b3)) || (b2 && !aligned16(b2))) {
        set_last_error("expert_ffn: pointers must be 16-byte aligned");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (row_end % 128 != 0 && row_end != rows_per_group) {
        set_last_error("expert_ffn: row_end must be a multiple of 128 or equal to rows_per_group");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (groups == 0 || row_end == row_begin) return ARISTOS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ARISTOS_DTYPE_BF16:
        case ARISTOS_DTYPE_F16:
        case ARISTOS_DTYPE_TF32:      // fp32 storage, tf32 tensor-core math
            return expert_ffn_tc_sm100(xg, count, groups, rows_per_group, experts, w1, w3, w2, b1, b3, b2, h_scratch, y,
                                       H, I, hidden_act,
                                       dtype == ARISTOS_DTYPE_BF16 ? 0 : (dtype == ARISTOS_DTYPE_F16 ? 1 : 2), row_begin,
                                       row_end, sm_limit, dev_status, st);
        case ARISTOS_DTYPE_F32:
            return expert_ffn_f32_simt(xg, count, groups, rows_per_group, experts, w1, w3, w2, b1, b3, b2, h_scratch, y, H, I,
                                       hidden_act, row_begin, row_end, st);
        default:
            set_last_error("expert_ffn: dtype %d not implemented (f32, tf32, bf16 and f16 are)", dtype);
            return ARISTOS_ERR_UNSUPPORTED;
    }
}

// ---- self-test of the bounded device-side wait ------------------------------------------------------------------------
namespace aristos {
namespace {
// One warp waits on an mbarrier that nothing ever arrives on, with the same wait routine the GEMM roles use; the wait
// must give up after limit_ns, report DEV_FAULT_TIMEOUT and let the kernel return normally.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, int32_t* dev_status, uint64_t* waited_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    const uint64_t t0 = ptx::globaltimer_ns();
    const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, dev_status, limit_ns);
    if (threadIdx.x == 0) *waited_ns = ok ? 0 : ptx::globaltimer_ns() - t0;
}
// The same for the wait on an arrival flag in global memory (what the up projection's producer does for every source
// rank in the expert-parallel layer): a flag word that nothing raises to `epoch`.
__global__ void bounded_flag_wait_selftest_kernel(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns,
                                                  int32_t* dev_status, uint64_t* waited_ns) {
    __shared__ int abort_flag;
    abort_flag = 0;
    __syncwarp();
    const uint64_t t0 = ptx::globaltimer_ns();
    bool ok = true;
    if (threadIdx.x == 0) ok = ptx::flag_wait_bounded(flag, epoch, &abort_flag, dev_status, limit_ns);
    if (threadIdx.x == 0) *waited_ns = ok ? 0 : ptx::globaltimer_ns() - t0;
}
}  // namespace
}  // namespace aristos

extern "C" int aristos_ffn_group_order(int position, int groups, int experts) {
    if (position < 0 || groups <= 0 || position >= groups) return -1;
    return ordered_group(position, groups, experts);
}

extern "C" int aristos_ffn_group_order_from(int position, int groups, int experts, int first_source) {
    if (position < 0 || groups <= 0 || position >= groups || experts <= 0 || first_source < 0 ||
        first_source >= (groups / experts > 0 ? groups / experts : 1))
        return -1;
    return ordered_group(position, groups, experts, first_source);
}

extern "C" aristos_status_t aristos_ffn_set_tile_mode(int mode) {
    if (mode < -1 || mode > 3) { set_last_error("ffn_set_tile_mode: mode must be -1 .. 3"); return ARISTOS_ERR_INVALID_ARG; }
    ffn_set_tile_mode(mode);
    return ARISTOS_OK;
}

extern "C" int aristos_ffn_tile_coord(int local, int row_tiles, int col_tiles, int band, int* row_tile, int* col_tile) {
    if (!row_tile || !col_tile || row_tiles < 1 || col_tiles < 1 || local < 0 || local >= row_tiles * col_tiles) return -1;
    band_tile_coord(local, row_tiles, col_tiles, band, row_tile, col_tile);
    return 0;
}

static aristos_status_t selftest_wait(int which, int limit_ms, int* waited_ms, void* stream);

extern "C" aristos_status_t aristos_selftest_bounded_wait(int limit_ms, int* waited_ms, void* stream) {
    return selftest_wait(0, limit_ms, waited_ms, stream);
}

extern "C" aristos_status_t aristos_selftest_bounded_flag_wait(int limit_ms, int* waited_ms, void* stream) {
    return selftest_wait(1, limit_ms, waited_ms, stream);
}

static aristos_status_t selftest_wait(int which, int limit_ms, int* waited_ms, void* stream) {
    if (limit_ms < 1 || limit_ms > 5000) { set_last_error("selftest: limit_ms must be in 1..5000"); return ARISTOS_ERR_INVALID_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int32_t* d_status = nullptr;
    ARISTOS_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&d_status), 32));
    uint64_t* d_waited = reinterpret_cast<uint64_t*>(d_status + 2);
    cudaError_t e = cudaMemsetAsync(d_status, 0, 32, st);
    if (e == cudaSuccess) {
        // the flag word (d_status + 4) stays 0; the wait asks for epoch 1
        if (which == 1)
            bounded_flag_wait_selftest_kernel<<<1, 32, 0, st>>>(reinterpret_cast<uint32_t*>(d_status + 4), 1u,
                                                                (uint64_t)limit_ms * 1000000ull, d_status, d_waited);
        else
            bounded_wait_selftest_kernel<<<1, 32, 0, st>>>((uint64_t)limit_ms * 1000000ull, d_status, d_waited);
        ARISTOS_COUNT_LAUNCH();
        e = cudaGetLastError();
    }
    int32_t bits = 0;
    uint64_t waited = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&bits, d_status, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&waited, d_waited, 8, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_status);
    if (e != cudaSuccess) return cuda_fail(e, "bounded-wait self-test");
    if (waited_ms) *waited_ms = (int)(waited / 1000000ull);
    if (bits & DEV_FAULT_TIMEOUT) { set_last_error("a bounded device-side wait expired (self-test)"); return ARISTOS_ERR_DEVICE_TIMEOUT; }
    return ARISTOS_OK;
}
