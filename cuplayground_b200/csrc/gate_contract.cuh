// Arithmetic of the gate's bit-exact logit contract, shared by the gate kernels: a row is consumed in 8-element
// chunks, even and odd elements accumulate separately with one fused multiply-add each.
#pragma once
#include "common.cuh"

namespace aristos {

constexpr int MAX_TOPK = 16;

// 8 consecutive elements as 4 (even, odd) pairs.
__device__ __forceinline__ void load8_pairs(const __nv_bfloat16* p, float2 (&v)[4]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
}
__device__ __forceinline__ void load8_pairs(const __half* p, float2 (&v)[4]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
}
__device__ __forceinline__ void load8_pairs(const float* p, float2 (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = make_float2(a.x, a.y); v[1] = make_float2(a.z, a.w);
    v[2] = make_float2(b.x, b.y); v[3] = make_float2(b.z, b.w);
}

// One 8-element chunk of a row in the form the FMA consumes: fp32 rows as four (even, odd) float2 pairs for the packed
// fp32x2 FMA; 16-bit rows as their four raw 32-bit words, multiplied by the mixed-precision FMA
// (fma.rn.f32.bf16 / .f16: 16-bit operands, fp32 accumulator, one rounding) so that nothing is unpacked on the
// integer pipe. Both give acc.x = fmaf(x[2i], w[2i], acc.x), acc.y = fmaf(x[2i+1], w[2i+1], acc.y).
template <typename T> struct GateChunk { uint32_t w[4]; };
template <> struct GateChunk<float> { float2 v[4]; };

__device__ __forceinline__ void load_chunk(const __nv_bfloat16* p, GateChunk<__nv_bfloat16>& c) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    c.w[0] = u.x; c.w[1] = u.y; c.w[2] = u.z; c.w[3] = u.w;
}
__device__ __forceinline__ void load_chunk(const __half* p, GateChunk<__half>& c) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    c.w[0] = u.x; c.w[1] = u.y; c.w[2] = u.z; c.w[3] = u.w;
}
__device__ __forceinline__ void load_chunk(const float* p, GateChunk<float>& c) { load8_pairs(p, c.v); }

__device__ __forceinline__ void fma_pair(float2& acc, const GateChunk<__nv_bfloat16>& x,
                                         const GateChunk<__nv_bfloat16>& w, int i) {
    asm("{\n\t"
        ".reg .b16 xl, xh, wl, wh;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "mov.b32 {wl, wh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, xl, wl, %0;\n\t"
        "fma.rn.f32.bf16 %1, xh, wh, %1;\n\t"
        "}"
        : "+f"(acc.x), "+f"(acc.y)
        : "r"(x.w[i]), "r"(w.w[i]));
}
__device__ __forceinline__ void fma_pair(float2& acc, const GateChunk<__half>& x, const GateChunk<__half>& w, int i) {
    asm("{\n\t"
        ".reg .b16 xl, xh, wl, wh;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "mov.b32 {wl, wh}, %3;\n\t"
        "fma.rn.f32.f16 %0, xl, wl, %0;\n\t"
        "fma.rn.f32.f16 %1, xh, wh, %1;\n\t"
        "}"
        : "+f"(acc.x), "+f"(acc.y)
        : "r"(x.w[i]), "r"(w.w[i]));
}
__device__ __forceinline__ void fma_pair(float2& acc, const GateChunk<float>& x, const GateChunk<float>& w, int i) {
    acc = __ffma2_rn(x.v[i], w.v[i], acc);
}

}  // namespace aristos
