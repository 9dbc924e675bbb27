// Combine: out[t] = sum_j w[t,j] * y[slot_of[t,j]], token-major, fixed j order, fp32 accumulation.
//
// Replaces Combine / VAA / deviceCombine of the reference (auditorium/combine.cuh:100-188, :19-93, :190-205), which
// scatters an expert-output tile into the owning tokens' rows with plain stores (k = 1) or vector atomicAdd
// (k > 1), unweighted, converting to float before accumulating (:24-31). Gathering per token instead of
// scattering per tile needs no atomics, so the sum has one fixed order and the result is deterministic; every
// access is a 16-byte load or store on a contiguous row.
#include "common.cuh"

namespace aristos {

template <typename T, int MAXK>
__global__ void __launch_bounds__(256)
combine_kernel(const T* __restrict__ y, const int32_t* __restrict__ slot_of, const float* __restrict__ topk_w,
               int S, int k, int H, T* __restrict__ out) {
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (t >= S) return;
    int slots[MAXK];
    float w[MAXK];
#pragma unroll
    for (int j = 0; j < MAXK; ++j) {
        slots[j] = (j < k) ? slot_of[(size_t)t * k + j] : -1;
        w[j] = (j < k) ? topk_w[(size_t)t * k + j] : 0.0f;
    }
    T* orow = out + (size_t)t * H;
    for (int c = lane * 8; c < H; c += 256) {
        float acc[8];
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[v] = 0.0f;
#pragma unroll
        for (int j = 0; j < MAXK; ++j) {
            if (slots[j] < 0) continue;
            float yv[8];
            load8(y + (size_t)slots[j] * H + c, yv);
#pragma unroll
            for (int v = 0; v < 8; ++v) acc[v] = fmaf(w[j], yv[v], acc[v]);
        }
        store8(orow + c, acc);
    }
}

template <typename T>
static aristos_status_t launch_combine(const void* y, const int32_t* slot_of, const float* w, int S, int k, int H,
                                       void* out, cudaStream_t st) {
    const int grid = ceil_div(S, 8);
    const T* yy = static_cast<const T*>(y);
    T* oo = static_cast<T*>(out);
    if (k <= 2) combine_kernel<T, 2><<<grid, 256, 0, st>>>(yy, slot_of, w, S, k, H, oo);
    else if (k <= 4) combine_kernel<T, 4><<<grid, 256, 0, st>>>(yy, slot_of, w, S, k, H, oo);
    else if (k <= 8) combine_kernel<T, 8><<<grid, 256, 0, st>>>(yy, slot_of, w, S, k, H, oo);
    else combine_kernel<T, 16><<<grid, 256, 0, st>>>(yy, slot_of, w, S, k, H, oo);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace aristos

using namespace aristos;

extern "C" aristos_status_t aristos_combine(const void* y, const int32_t* slot_of, const float* topk_w, int S, int k,
                                            int H, int dtype, void* out, void* stream) {
    if (!y || !slot_of || !topk_w || !out) { set_last_error("combine: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (S < 0 || k <= 0 || k > 16 || H <= 0 || H % 8 != 0) { set_last_error("combine: bad size (H %% 8 == 0, k <= 16)"); return ARISTOS_ERR_INVALID_ARG; }
    if (!aligned16(y) || !aligned16(out)) { set_last_error("combine: pointers must be 16-byte aligned"); return ARISTOS_ERR_INVALID_ARG; }
    if (S == 0) return ARISTOS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ARISTOS_DTYPE_F32:
        case ARISTOS_DTYPE_TF32: return launch_combine<float>(y, slot_of, topk_w, S, k, H, out, st);
        case ARISTOS_DTYPE_BF16: return launch_combine<__nv_bfloat16>(y, slot_of, topk_w, S, k, H, out, st);
        case ARISTOS_DTYPE_F16: return launch_combine<__half>(y, slot_of, topk_w, S, k, H, out, st);
        default:
            set_last_error("combine: dtype %d not implemented (f32, bf16 and f16 are)", dtype);
            return ARISTOS_ERR_UNSUPPORTED;
    }
}
