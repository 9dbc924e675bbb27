// Internal helpers shared by the kernels and the host code of libaristos_moe.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aristos_moe.h"

namespace aristos {

// Bits OR-ed into the device status word by kernels; mapped to aristos_status_t by the host.
enum : int32_t { DEV_FAULT_TIMEOUT = 1, DEV_FAULT_BOUNDS = 2, DEV_FAULT_SCREEN = 4, DEV_FAULT_NONFINITE = 8 };

void set_last_error(const char* fmt, ...);
aristos_status_t cuda_fail(cudaError_t e, const char* what);

#define ARISTOS_CUDA_TRY(expr)                                                  \
    do {                                                                        \
        cudaError_t _e = (expr);                                                \
        if (_e != cudaSuccess) return ::aristos::cuda_fail(_e, #expr);          \
    } while (0)

#define ARISTOS_TRY(expr)                                                       \
    do {                                                                        \
        aristos_status_t _s = (expr);                                           \
        if (_s != ARISTOS_OK) return _s;                                        \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t dtype_bytes(int dtype) {
    switch (dtype) {
        case ARISTOS_DTYPE_F32: case ARISTOS_DTYPE_TF32: return 4;
        case ARISTOS_DTYPE_BF16: case ARISTOS_DTYPE_F16: return 2;
        case ARISTOS_DTYPE_FP8_E4M3: return 1;
        default: return 0;
    }
}
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Row groups are numbered source-major (g = source * experts + expert). The GEMM kernels walk them expert-major
// (position v -> expert v / sources, source v % sources), so that the tiles of all the groups that use one expert's
// weights run back to back and the weights stay in L2 instead of being streamed once per source rank.
#ifdef __CUDACC__
__host__ __device__
#endif
// Within an expert the sources are taken in ring order starting at first_source: a rank starts with the rows it
// gathered itself, which are in its memory before the kernel launches, while the peers' rows are still arriving.
inline int ordered_group(int v, int groups, int experts, int first_source = 0) {
    const int sources = experts > 0 ? groups / experts : 0;
    if (sources <= 1 || sources * experts != groups) return v;
    const int e = v / sources;
    int s = v - e * sources + first_source;
    if (s >= sources) s -= sources;
    return s * experts + e;
}

// Order of the tiles of one row group: mt row tiles x nt column tiles, `local` in [0, mt * nt). The row tiles are cut
// into bands of `band` row tiles; inside a band the row tile runs fastest, then the column tile, then the next band.
// The CTAs that run at the same time then share `band` A panels and about (CTAs / band) B panels, instead of all mt
// A panels and few B panels. band >= mt gives the plain row-tile-fastest order.
#ifdef __CUDACC__
__host__ __device__
#endif
inline void band_tile_coord(int local, int mt, int nt, int band, int* m, int* n) {
    if (band <= 0 || band >= mt) { *m = local % mt; *n = local / mt; return; }
    const int per_band = band * nt;
    const int full = mt / band;
    if (local < full * per_band) {
        const int b = local / per_band, r = local - b * per_band;
        *n = r / band;
        *m = b * band + (r - *n * band);
    } else {
        const int rem = mt - full * band, r = local - full * per_band;
        *n = r / rem;
        *m = full * band + (r - *n * rem);
    }
}
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Number of SMs of the current device (cached per device).
int device_sm_count();

// Per-thread launch counter, read by the layer to report how many kernels it launched.
int64_t& launch_counter();
#define ARISTOS_COUNT_LAUNCH() (++::aristos::launch_counter())

#ifdef __CUDACC__
// ---- device-side loads of the two storage types as fp32 ---------------------------------------------------------
// 8 consecutive elements starting at p (16 B for bf16, 32 B for fp32).
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t*>(&t);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void store8(__half* p, const float (&v)[8]) {
    uint4 u;
    __half2 t;
    t = __floats2half2_rn(v[0], v[1]); u.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2half2_rn(v[2], v[3]); u.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2half2_rn(v[4], v[5]); u.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2half2_rn(v[6], v[7]); u.w = *reinterpret_cast<uint32_t*>(&t);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

__device__ __forceinline__ float act_relu(float v) { return v > 0.0f ? v : 0.0f; }
__device__ __forceinline__ float act_gelu(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f)); }
__device__ __forceinline__ float act_silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
#endif

}  // namespace aristos
