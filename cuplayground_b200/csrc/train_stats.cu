// Training-mode pieces of the layer (is_training = 1 in aristos_config.json; the reference's schema has the flag,
// aristos_config.schema.json:20-23, and no code behind it): per-expert load-balance statistics of a forward's routing,
// the ingredients of the usual auxiliary loss, computed on the device from the gate's outputs.
//
//   frac[e]  = share of the S*k assignments that chose expert e (before capacity drops)
//   prob[e]  = (sum of the gate weights given to e) / S
//   aux      = E * sum_e frac[e] * prob[e]
//   dropped  = share of the assignments that capacity dropped
// Layout of the output: [frac (E) | prob (E) | aux | dropped], fp32.
//
// One CTA per expert walks all assignments in a fixed order (thread i takes assignments i, i + 256, ... in turn, then
// a fixed tree over the 256 partial sums), so the float sums do not depend on scheduling: two runs give the same bits.
#include "common.cuh"

namespace aristos {

namespace {

constexpr int LB_THREADS = 256;

__global__ void __launch_bounds__(LB_THREADS)
load_balance_expert_kernel(const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
                           const int32_t* __restrict__ slot_of, int n, int S, int E, float* __restrict__ stats) {
    __shared__ float s_w[LB_THREADS];
    __shared__ int s_c[LB_THREADS];
    __shared__ int s_d[LB_THREADS];
    const int e = blockIdx.x;
    float w = 0.0f;
    int c = 0, d = 0;
    for (int i = threadIdx.x; i < n; i += LB_THREADS) {
        if (topk_idx[i] == e) {
            w += topk_w[i];
            c += 1;
            d += slot_of[i] < 0 ? 1 : 0;
        }
    }
    s_w[threadIdx.x] = w;
    s_c[threadIdx.x] = c;
    s_d[threadIdx.x] = d;
    __syncthreads();
    for (int half = LB_THREADS / 2; half >= 1; half >>= 1) {
        if ((int)threadIdx.x < half) {
            s_w[threadIdx.x] += s_w[threadIdx.x + half];
            s_c[threadIdx.x] += s_c[threadIdx.x + half];
            s_d[threadIdx.x] += s_d[threadIdx.x + half];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        stats[e] = (float)s_c[0] / (float)n;
        stats[E + e] = s_w[0] / (float)S;
        // per-expert dropped counts are parked behind the public layout for the finishing kernel
        reinterpret_cast<int32_t*>(stats + 2 * E + 2)[e] = s_d[0];
    }
}

// aux and dropped from the per-expert values, in expert order (one thread: E <= 1024 terms).
__global__ void load_balance_finish_kernel(int n, int E, float* __restrict__ stats) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float aux = 0.0f;
    int dropped = 0;
    for (int e = 0; e < E; ++e) {
        aux = fmaf(stats[e], stats[E + e], aux);
        dropped += reinterpret_cast<const int32_t*>(stats + 2 * E + 2)[e];
    }
    stats[2 * E] = aux * (float)E;
    stats[2 * E + 1] = (float)dropped / (float)n;
}

}  // namespace

}  // namespace aristos

using namespace aristos;

extern "C" size_t aristos_load_balance_stats_bytes(int E) {
    return E > 0 ? align_up((size_t)(3 * E + 2) * sizeof(float), 256) : 0;
}

extern "C" aristos_status_t aristos_load_balance_stats(const int32_t* topk_idx, const float* topk_w,
                                                       const int32_t* slot_of, int S, int k, int E, float* stats,
                                                       void* stream) {
    if (!topk_idx || !topk_w || !slot_of || !stats) { set_last_error("load_balance_stats: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (S <= 0 || k <= 0 || E <= 0 || E > 1024 || (int64_t)S * k > 0x7fffffffLL) {
        set_last_error("load_balance_stats: bad size");
        return ARISTOS_ERR_INVALID_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    load_balance_expert_kernel<<<E, LB_THREADS, 0, st>>>(topk_idx, topk_w, slot_of, S * k, S, E, stats);
    ARISTOS_COUNT_LAUNCH();
    load_balance_finish_kernel<<<1, 32, 0, st>>>(S * k, E, stats);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}
