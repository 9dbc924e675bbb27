// Internal entry points of the expert FFN (behind aristos_expert_ffn*; also called by the layer).
#pragma once
#include "common.cuh"

namespace aristos {

// Expert-parallel arguments of the tensor-core FFN (all optional).
struct FfnEpArgs {
    // peer_world > 0: the down projection's output tiles are stored straight into the source ranks' return buffers
    // peer_y[0 .. peer_world) (each (peer_world * experts, rows_per_group, H)) instead of y: group g = src * experts + e
    // goes to peer_y[src], block peer_rank * experts + e.
    void* const* peer_y = nullptr;
    int peer_world = 0;
    int peer_rank = 0;
    // Source order inside an expert starts at this rank (own rows first).
    int first_source = 0;
    // src_flags != nullptr: the up projection waits, per source rank, until src_flags[src] has reached flag_epoch
    // before it loads that rank's rows (bounded by flag_limit_ms, 0 = 2000; expiry reports DEV_FAULT_TIMEOUT).
    const uint32_t* src_flags = nullptr;
    uint32_t flag_epoch = 0;
    uint32_t flag_limit_ms = 0;
    int self_source = -1;     // rows of this source rank are complete before the launch: no flag wait for them
    // Counter scratch (device, groups * ceil(rows / 128) int32): with it, small row groups run the up and the down
    // projection as ONE persistent launch whose down tiles wait for the up tiles of their row tile.
    int32_t* updown_scratch = nullptr;
    size_t updown_scratch_ints = 0;
};

// bf16 / fp16 / tf32 on the tensor cores (fmt 0 / 1 / 2).
aristos_status_t expert_ffn_tc_sm100(const void* xg, const int32_t* count, int groups, int rows_per_group,
                                     int experts, const void* w1, const void* w3, const void* w2, const void* b1,
                                     const void* b3, const void* b2, void* h_scratch, void* y, int H, int I,
                                     int hidden_act, int fmt, int row_begin, int row_end, int sm_limit,
                                     int32_t* dev_status, cudaStream_t st, const FfnEpArgs* ep = nullptr);
// Tile shape of the tensor-core FFN: 0 automatic, 1 single-CTA tiles, 2 CTA pairs + single-CTA tail, 3 CTA pairs with
// every group padded to 256 rows; anything else re-reads ARISTOS_FFN_TILES.
void ffn_set_tile_mode(int mode);
int ffn_tile_mode();
aristos_status_t expert_ffn_f32_simt(const void* xg, const int32_t* count, int groups, int rows_per_group, int experts,
                                     const void* w1, const void* w3, const void* w2, const void* b1, const void* b3,
                                     const void* b2, void* h_scratch, void* y, int H, int I, int hidden_act,
                                     int row_begin, int row_end, cudaStream_t st);
aristos_status_t expert_ffn_fp8_sm100(const void* xq, const float* sx, const int32_t* count, int groups,
                                      int rows_per_group, int experts, const void* w1q, const float* s1,
                                      const void* w3q, const float* s3, const void* w2q, const float* s2, void* h,
                                      void* hq, float* sh, void* y, int H, int I, int hidden_act, int row_begin,
                                      int row_end, int sm_limit, int32_t* dev_status, cudaStream_t st,
                                      void* const* peer_y = nullptr, int peer_world = 0, int peer_rank = 0,
                                      const int32_t* dense_src_off = nullptr, int dense_ret_rows = 0);
// (the fp8 variant takes the peer output arguments directly; dense_src_off != nullptr: one dense group per expert that
// holds every source rank's rows, see dense_exchange_plan in ep_kernels.h)

}  // namespace aristos
