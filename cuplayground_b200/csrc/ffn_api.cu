// aristos_expert_ffn: argument checks and the per-dtype kernels behind the C ABI.
#include "common.cuh"

namespace aristos {
aristos_status_t expert_ffn_bf16_sm100(const void* xg, const int32_t* count, int groups, int rows_per_group,
                                       int experts, const void* w1, const void* w3, const void* w2, void* h_scratch,
                                       void* y, int H, int I, int hidden_act, int row_begin, int row_end,
                                       int sm_limit, int32_t* dev_status, cudaStream_t st);
aristos_status_t expert_ffn_f32_simt(const void* xg, const int32_t* count, int groups, int rows_per_group, int experts,
                                     const void* w1, const void* w3, const void* w2, void* h_scratch, void* y, int H,
                                     int I, int hidden_act, int row_begin, int row_end, cudaStream_t st);
}  // namespace aristos

using namespace aristos;

extern "C" aristos_status_t aristos_expert_ffn(const void* xg, const int32_t* count, int groups, int rows_per_group,
                                               int experts, const void* w1, const void* w3, const void* w2,
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
        (w3 && !aligned16(w3))) {
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
            return expert_ffn_bf16_sm100(xg, count, groups, rows_per_group, experts, w1, w3, w2, h_scratch, y, H, I,
                                         hidden_act, row_begin, row_end, sm_limit, dev_status, st);
        case ARISTOS_DTYPE_F32:
            return expert_ffn_f32_simt(xg, count, groups, rows_per_group, experts, w1, w3, w2, h_scratch, y, H, I,
                                       hidden_act, row_begin, row_end, st);
        default:
            set_last_error("expert_ffn: dtype %d not implemented (f32 and bf16 are)", dtype);
            return ARISTOS_ERR_UNSUPPORTED;
    }
}
