// Gate: logits = x * Wg^T (+ bias) in fp32 with a fixed reduction order, top-k on the logits, softmax / sigmoid
// combine weights.
//
// The reference has no gate (its only trace is the unused gateScratch array, benchmarks.cuh:168-178); operand
// layout follows its expert-tile contract: x (S,H) row-major, Wg (E,H) row-major = the (N,K) B operand of
// mma.cuh:396-397.
//
// Bit-exact contract (mirrored by the CPU oracle): for a token t and expert e, lane c of a warp accumulates
//   p[c] = fmaf(x[t,h], Wg[e,h], p[c])   over the 8-element chunks q = h/8 with q % 32 == c, in increasing h,
// then the 32 partial sums are combined by the xor butterfly 16, 8, 4, 2, 1 and the bias is added last.
// Products of bf16 values are exact in fp32, every step is one IEEE operation, so the logits do not depend on
// the launch geometry and the CPU reproduces them bit for bit. Top-k is taken on the logits (exp is monotone, so
// the selected indices cannot depend on its rounding); ties go to the lower expert index.
#include "common.cuh"

namespace aristos {

constexpr int GATE_WARPS = 8;   // warps per CTA
constexpr int GATE_TT = 4;      // tokens per warp pass
constexpr int GATE_TE = 8;      // experts per register tile
constexpr int MAX_TOPK = 16;

template <typename T>
__global__ void __launch_bounds__(GATE_WARPS * 32)
gate_topk_kernel(const T* __restrict__ x, const T* __restrict__ wg, const float* __restrict__ bias, int S, int H,
                 int E, int k, int gate_fn, int renorm, int32_t* __restrict__ topk_idx,
                 float* __restrict__ topk_w, float* __restrict__ logits_out) {
    extern __shared__ float s_logits[];  // [GATE_WARPS][GATE_TT][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = (blockIdx.x * GATE_WARPS + warp) * GATE_TT;
    if (t0 >= S) return;
    float* my_logits = s_logits + (size_t)warp * GATE_TT * E;
    const int nchunk = H >> 3;

    const T* xrow[GATE_TT];
#pragma unroll
    for (int tt = 0; tt < GATE_TT; ++tt) xrow[tt] = x + (size_t)min(t0 + tt, S - 1) * H;

    for (int e0 = 0; e0 < E; e0 += GATE_TE) {
        float acc[GATE_TT][GATE_TE];
#pragma unroll
        for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
            for (int ee = 0; ee < GATE_TE; ++ee) acc[tt][ee] = 0.0f;
        const T* wrow[GATE_TE];
#pragma unroll
        for (int ee = 0; ee < GATE_TE; ++ee) wrow[ee] = wg + (size_t)min(e0 + ee, E - 1) * H;

        for (int q = lane; q < nchunk; q += 32) {
            float xv[GATE_TT][8];
#pragma unroll
            for (int tt = 0; tt < GATE_TT; ++tt) load8(xrow[tt] + q * 8, xv[tt]);
#pragma unroll
            for (int ee = 0; ee < GATE_TE; ++ee) {
                float wv[8];
                load8(wrow[ee] + q * 8, wv);
#pragma unroll
                for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
                    for (int v = 0; v < 8; ++v) acc[tt][ee] = fmaf(xv[tt][v], wv[v], acc[tt][ee]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
            for (int ee = 0; ee < GATE_TE; ++ee) {
                float p = acc[tt][ee];
#pragma unroll
                for (int m = 16; m >= 1; m >>= 1) p = p + __shfl_xor_sync(0xffffffffu, p, m);
                const int e = e0 + ee;
                if (e < E) {
                    if (bias) p = p + bias[e];
                    if (lane == 0) my_logits[tt * E + e] = p;
                }
            }
    }
    __syncwarp();

    for (int tt = 0; tt < GATE_TT; ++tt) {
        const int t = t0 + tt;
        if (t >= S) break;
        const float* l = my_logits + tt * E;
        if (logits_out)
            for (int e = lane; e < E; e += 32) logits_out[(size_t)t * E + e] = l[e];
        int chosen[MAX_TOPK];
        float chosen_l[MAX_TOPK];
#pragma unroll 1
        for (int j = 0; j < k; ++j) {
            float bv = 0.0f;
            int bi = -1;
            for (int e = lane; e < E; e += 32) {
                bool taken = false;
                for (int i = 0; i < j; ++i) taken |= (chosen[i] == e);
                if (taken) continue;
                const float v = l[e];
                if (bi < 0 || v > bv) { bv = v; bi = e; }   // strict '>' keeps the lowest index within a lane
            }
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
                const bool take = (oi >= 0) && (bi < 0 || ov > bv || (ov == bv && oi < bi));
                if (take) { bv = ov; bi = oi; }
            }
            chosen[j] = bi;
            chosen_l[j] = bv;
        }
        float w_sel[MAX_TOPK];
        if (gate_fn == ARISTOS_GATE_SOFTMAX) {
            const float mx = chosen_l[0];
            float den = 0.0f;
            for (int e = lane; e < E; e += 32) den += expf(l[e] - mx);
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) den += __shfl_xor_sync(0xffffffffu, den, m);
            for (int j = 0; j < k; ++j) w_sel[j] = expf(chosen_l[j] - mx) / den;
        } else {
            for (int j = 0; j < k; ++j) w_sel[j] = 1.0f / (1.0f + expf(-chosen_l[j]));
        }
        if (renorm) {
            float s = 0.0f;
            for (int j = 0; j < k; ++j) s += w_sel[j];
            for (int j = 0; j < k; ++j) w_sel[j] = w_sel[j] / s;
        }
        for (int j = 0; j < k; ++j)
            if (lane == j) {
                topk_idx[(size_t)t * k + j] = chosen[j];
                topk_w[(size_t)t * k + j] = w_sel[j];
            }
    }
}

template <typename T>
static aristos_status_t launch_gate(const void* x, const void* wg, const float* bias, int S, int H, int E, int k,
                                    int gate_fn, int renorm, int32_t* topk_idx, float* topk_w, float* logits_out,
                                    cudaStream_t stream) {
    const size_t smem = sizeof(float) * GATE_WARPS * GATE_TT * (size_t)E;
    if (smem > 48 * 1024)
        ARISTOS_CUDA_TRY(cudaFuncSetAttribute(gate_topk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)smem));
    const int grid = ceil_div(S, GATE_WARPS * GATE_TT);
    gate_topk_kernel<T><<<grid, GATE_WARPS * 32, smem, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(wg), bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w,
        logits_out);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace aristos

using namespace aristos;

extern "C" aristos_status_t aristos_gate_topk(const void* x, const void* w_gate, const float* gate_bias, int S,
                                              int H, int E, int k, int gate_fn, int renorm, int dtype,
                                              int32_t* topk_idx, float* topk_w, float* logits_out, void* stream) {
    if (!x || !w_gate || !topk_idx || !topk_w) { set_last_error("gate: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (S < 0 || H <= 0 || E <= 0 || k <= 0) { set_last_error("gate: bad size"); return ARISTOS_ERR_INVALID_ARG; }
    if (H % 8 != 0 || k > E || k > MAX_TOPK || E > 1024) {
        set_last_error("gate: need H %% 8 == 0, k <= min(E, %d), E <= 1024", MAX_TOPK);
        return ARISTOS_ERR_CONFIG;
    }
    if (!aligned16(x) || !aligned16(w_gate)) { set_last_error("gate: pointers must be 16-byte aligned"); return ARISTOS_ERR_INVALID_ARG; }
    if (gate_fn != ARISTOS_GATE_SOFTMAX && gate_fn != ARISTOS_GATE_SIGMOID) return ARISTOS_ERR_INVALID_ARG;
    if (S == 0) return ARISTOS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ARISTOS_DTYPE_F32:
            return launch_gate<float>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, st);
        case ARISTOS_DTYPE_BF16:
            return launch_gate<__nv_bfloat16>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, st);
        default:
            set_last_error("gate: dtype %d not implemented (f32 and bf16 are)", dtype);
            return ARISTOS_ERR_UNSUPPORTED;
    }
}
