// Synthetic inputs: Philox4x32-10 + Box-Muller normal fill on the device.
// The reference draws its test inputs from Philox as well (main.cu:22-31, cuRAND Philox4_32_10). Element i uses
// counter (i/4, 0, stream_id, 0), key = seed and output word i%4, so a tensor's values do not depend on the launch
// geometry. The CPU oracle implements the same generator; the two agree up to the rounding of logf/sinf/cosf.
#include "common.cuh"

namespace aristos {
namespace {

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ dst, int64_t n, float mean, float std, uint32_t k0, uint32_t k1,
                                   uint32_t stream_id) {
    const int64_t nblk = (n + 3) / 4;
    for (int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; b < nblk; b += (int64_t)gridDim.x * blockDim.x) {
        uint32_t c[4] = {(uint32_t)b, (uint32_t)((uint64_t)b >> 32), stream_id, 0u};
        philox4x32_10(c, k0, k1);
        float z[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float u1 = ((float)(c[2 * h] >> 8) + 1.0f) * (1.0f / 16777216.0f);
            const float u2 = (float)(c[2 * h + 1] >> 8) * (1.0f / 16777216.0f);
            const float r = sqrtf(-2.0f * logf(u1));
            float sn, cs;
            sincosf(6.283185307179586f * u2, &sn, &cs);
            z[2 * h] = r * cs;
            z[2 * h + 1] = r * sn;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t i = 4 * b + j;
            if (i < n) dst[i] = static_cast<T>(mean + std * z[j]);
        }
    }
}

}  // namespace
}  // namespace aristos

using namespace aristos;

extern "C" aristos_status_t aristos_fill_normal(void* dst, int64_t n, float mean, float std, uint64_t seed,
                                                uint32_t stream_id, int dtype, void* stream) {
    if (!dst || n < 0) { set_last_error("fill_normal: bad argument"); return ARISTOS_ERR_INVALID_ARG; }
    if (n == 0) return ARISTOS_OK;
    const int64_t nblk = (n + 3) / 4;
    const int grid = (int)((nblk + 255) / 256 < 148 * 16 ? (nblk + 255) / 256 : 148 * 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    if (dtype == ARISTOS_DTYPE_F32 || dtype == ARISTOS_DTYPE_TF32) fill_normal_kernel<float><<<grid, 256, 0, st>>>((float*)dst, n, mean, std, k0, k1, stream_id);
    else if (dtype == ARISTOS_DTYPE_BF16) fill_normal_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)dst, n, mean, std, k0, k1, stream_id);
    else if (dtype == ARISTOS_DTYPE_F16) fill_normal_kernel<__half><<<grid, 256, 0, st>>>((__half*)dst, n, mean, std, k0, k1, stream_id);
    else { set_last_error("fill_normal: dtype %d not implemented", dtype); return ARISTOS_ERR_UNSUPPORTED; }
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}
