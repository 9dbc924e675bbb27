// Internal entry points of the expert FFN (behind aristos_expert_ffn*; also called by the layer).
#pragma once
#include "common.cuh"

namespace aristos {

// bf16 / fp16 / tf32 on the tensor cores (fmt 0 / 1 / 2); the fp8 variant takes the same peer arguments. With peer_world > 0 the down projection's output tiles are
// stored straight into the source ranks' return buffers peer_y[0 .. peer_world) (each (peer_world * experts,
// rows_per_group, H)) instead of y: group g = src * experts + e goes to peer_y[src], block peer_rank * experts + e.
aristos_status_t expert_ffn_tc_sm100(const void* xg, const int32_t* count, int groups, int rows_per_group,
                                     int experts, const void* w1, const void* w3, const void* w2, const void* b1,
                                     const void* b3, const void* b2, void* h_scratch, void* y, int H, int I,
                                     int hidden_act, int fmt, int row_begin, int row_end, int sm_limit,
                                     int32_t* dev_status, cudaStream_t st, void* const* peer_y = nullptr,
                                     int peer_world = 0, int peer_rank = 0);
aristos_status_t expert_ffn_f32_simt(const void* xg, const int32_t* count, int groups, int rows_per_group, int experts,
                                     const void* w1, const void* w3, const void* w2, const void* b1, const void* b3,
                                     const void* b2, void* h_scratch, void* y, int H, int I, int hidden_act,
                                     int row_begin, int row_end, cudaStream_t st);
aristos_status_t expert_ffn_fp8_sm100(const void* xq, const float* sx, const int32_t* count, int groups,
                                      int rows_per_group, int experts, const void* w1q, const float* s1,
                                      const void* w3q, const float* s3, const void* w2q, const float* s2, void* h,
                                      void* hq, float* sh, void* y, int H, int I, int hidden_act, int row_begin,
                                      int row_end, int sm_limit, int32_t* dev_status, cudaStream_t st,
                                      void* const* peer_y = nullptr, int peer_world = 0, int peer_rank = 0);

}  // namespace aristos
