// Expert FFN for fp32 tensors (torch_dtype 0): a shared-memory tiled SIMT GEMM with the fused epilogue.
//
// fp32 results must agree with an fp32 recomputation to 1e-4 relative, which rules out tensor-core TF32 inputs, so
// this path uses FFMA like the reference does for fp32 (its generic MMAConfig falls back to UniversalFMA,
// processor/tiling.cuh:97-104, under the same C = act(A * B^T) tile contract, mma.cuh:46-161). It serves the
// small fp32 reference configuration; the bf16 path is ffn_sm100.cu.
#include "common.cuh"

namespace aristos {
namespace {

constexpr int TS = 64;   // tile rows / cols
constexpr int TK = 16;   // K slab

// out[g, r, n] = epi( sum_k A[g, r, k] * B0[e, n, k] [, sum_k A[g, r, k] * B1[e, n, k]] )
__global__ void __launch_bounds__(256)
ffn_simt_kernel(const float* __restrict__ A, const float* __restrict__ B0, const float* __restrict__ B1,
                const float* __restrict__ bias0, const float* __restrict__ bias1, const int32_t* __restrict__ count, int experts, int rows_per_group, int row_begin, int row_end, int N,
                int K, int gated, int act, float* __restrict__ out) {
    const int g = blockIdx.z;
    const int m0 = row_begin + blockIdx.y * TS;
    const int row_limit = min(count[g], row_end);
    if (m0 >= row_limit) return;
    const int n0 = blockIdx.x * TS;
    const int e = g % experts;
    __shared__ float sA[TK][TS + 1], sB0[TK][TS + 1], sB1[TK][TS + 1];
    const float* Ag = A + (size_t)g * rows_per_group * K;
    const float* B0e = B0 + (size_t)e * N * K;
    const float* B1e = gated ? B1 + (size_t)e * N * K : nullptr;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
    float acc0[4][4] = {}, acc1[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int i = threadIdx.x; i < TS * TK; i += 256) {
            const int r = i / TK, kk = i % TK;
            const int row = m0 + r, col = n0 + r;
            sA[kk][r] = (row < row_limit) ? Ag[(size_t)row * K + k0 + kk] : 0.0f;
            sB0[kk][r] = (col < N) ? B0e[(size_t)col * K + k0 + kk] : 0.0f;
            if (gated) sB1[kk][r] = (col < N) ? B1e[(size_t)col * K + k0 + kk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b0[4], b1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = sA[kk][ty * 4 + i];
                b0[i] = sB0[kk][tx * 4 + i];
                b1[i] = gated ? sB1[kk][tx * 4 + i] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc0[i][j] = fmaf(a[i], b0[j], acc0[i][j]);
                    if (gated) acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = m0 + ty * 4 + i;
        if (row >= row_limit) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + tx * 4 + j;
            if (col >= N) continue;
            float v = acc0[i][j];
            if (bias0) v += bias0[(size_t)e * N + col];
            if (gated) {
                float u = acc1[i][j];
                if (bias1) u += bias1[(size_t)e * N + col];
                v = (v / (1.0f + expf(-v))) * u;
            }
            else if (act == ARISTOS_ACT_RELU) v = act_relu(v);
            else if (act == ARISTOS_ACT_GELU) v = act_gelu(v);
            out[((size_t)g * rows_per_group + row) * N + col] = v;
        }
    }
}

}  // namespace

aristos_status_t expert_ffn_f32_simt(const void* xg, const int32_t* count, int groups, int rows_per_group, int experts,
                                     const void* w1, const void* w3, const void* w2, const void* b1, const void* b3,
                                     const void* b2, void* h_scratch, void* y, int H, int I, int hidden_act,
                                     int row_begin, int row_end, cudaStream_t st) {
    if (groups > 65535) { set_last_error("expert_ffn(f32): too many groups"); return ARISTOS_ERR_CONFIG; }
    if (H % TK != 0 || I % TK != 0) { set_last_error("expert_ffn(f32): H and I must be multiples of 16"); return ARISTOS_ERR_CONFIG; }
    const int mt = ceil_div(row_end - row_begin, TS);
    if (mt <= 0 || groups <= 0) return ARISTOS_OK;
    const bool gated = hidden_act == ARISTOS_ACT_SWIGLU;
    dim3 g1(ceil_div(I, TS), mt, groups), g2(ceil_div(H, TS), mt, groups);
    ffn_simt_kernel<<<g1, 256, 0, st>>>((const float*)xg, (const float*)w1, (const float*)w3, (const float*)b1,
                                        gated ? (const float*)b3 : nullptr, count, experts,
                                        rows_per_group, row_begin, row_end, I, H, gated ? 1 : 0, hidden_act,
                                        (float*)h_scratch);
    ARISTOS_COUNT_LAUNCH();
    ffn_simt_kernel<<<g2, 256, 0, st>>>((const float*)h_scratch, (const float*)w2, nullptr, (const float*)b2, nullptr,
                                        count, experts,
                                        rows_per_group, row_begin, row_end, H, I, 0, ARISTOS_ACT_IDENTITY, (float*)y);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace aristos
