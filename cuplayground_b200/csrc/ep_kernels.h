// Kernels that move rows between ranks by storing through peer pointers (see ep_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/aristos_moe.h"

namespace aristos {

struct PeerPtrs {
    void* p[16];   // rank r's copy of one exchange buffer, as mapped into this process
};

// Dispatch without a staging buffer: token row t goes, for each kept assignment whose position inside its expert lies
// in [pos_lo, pos_hi), into the buffer of the rank that owns the expert. With count != nullptr the same launch also
// stores count[0 .. E) into the owners' received-count lists (count_dst: every rank's list), entry
// src_rank * E_local + e % E_local.
aristos_status_t permute_rows_to_peers(const void* x, const int32_t* slot_of, int S, int k, size_t row_bytes,
                                       int E_local, int cap, int src_rank, int pos_lo, int pos_hi, const PeerPtrs& dst,
                                       cudaStream_t st, const int32_t* count = nullptr, int E = 0,
                                       const PeerPtrs* count_dst = nullptr, const int32_t* send_base = nullptr,
                                       int group_rows = 0, int dest_filter = 0);
// dest_filter: 0 every kept row, 1 only the rows whose expert this rank owns (a local copy), 2 only the rows that go
// to other ranks (what can run beside the expert GEMM while it works on the local rows).
// Dense packing of the received rows per expert across source ranks. From allcount[src * E + e] (every rank's counts
// of every expert): send_base[e] = where this rank's rows start in expert e's group at its owner (the lower ranks'
// rows come first); for this rank's experts dense_count[el] = rows received in all and src_off[el * (world + 1) + s]
// = first row of source s (entry `world` = the total). With send_base given, permute_rows_to_peers stores row pos of
// expert e at row el * group_rows + send_base[e] + pos of the owner's buffer.
aristos_status_t dense_exchange_plan(const int32_t* allcount, int world, int E, int E_local, int rank,
                                     int32_t* send_base, int32_t* dense_count, int32_t* src_off, cudaStream_t st);
// Valid rows [row_lo, row_hi) of the local expert outputs (groups x cap rows, count[g] valid) back into their source
// ranks' buffers.
aristos_status_t return_rows_to_peers(const void* y, const int32_t* count, int groups, int E_local, int cap,
                                      size_t row_bytes, int this_rank, int row_lo, int row_hi, const PeerPtrs& dst,
                                      cudaStream_t st);

}  // namespace aristos
