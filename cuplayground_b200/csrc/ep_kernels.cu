// Expert-parallel exchange done by kernels that store straight into the destination GPU's memory (peer pointers
// over NVLink): the gather of token rows IS the dispatch all-to-all, and the return of expert outputs copies only
// the rows that exist. Used where padded fixed-size blocks would move far more than the kept rows (drop-free
// routing, capacity = tokens).
//
// Reference counterpart: the commented peer-store GEMM (mma.cuh:445-539 writes its C tile into another GPU's memory
// after cudaDeviceEnablePeerAccess) and the put-with-signal of auditorium/overlap.cuh:94-136. Arrival is published
// afterwards by the epoch flags of ep_p2p.cu; nothing here waits on a peer.
#include "common.cuh"
#include "ep_kernels.h"

namespace aristos {

namespace {

// Token-major gather into the owners' buffers: assignment (t, j) with slot e*cap + pos goes to rank e / E_local, row
// ((src_rank*E_local + e % E_local)*cap + pos) of that rank's buffer; only positions in [pos_lo, pos_hi) are handled
// (one row window of the pipeline). One warp per token, 16-byte lanes. With count != nullptr the kernel also stores
// the per-expert row counts into the owners' count lists (the same stream order publishes both).
// With send_base != nullptr the destination is densely packed per expert: all sources' rows of expert e follow each
// other in one group of group_rows rows, this rank's rows starting at row send_base[e] (the rows of the lower ranks
// come first), so the owner computes whole tiles of one expert instead of one padded group per (source, expert).
template <int MAXK>
__global__ void __launch_bounds__(256)
permute_rows_peer_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ slot_of, int S, int k, int row_vec,
                         int E_local, int cap, int src_rank, int pos_lo, int pos_hi, PeerPtrs dst,
                         const int32_t* __restrict__ count, int E, PeerPtrs count_dst,
                         const int32_t* __restrict__ send_base, int group_rows, int dest_filter) {
    // the first CTA also delivers the row counts: count[e] becomes entry (src_rank, e % E_local) of the owner's list
    if (count != nullptr && blockIdx.x == 0)
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            const int owner = e / E_local;
            static_cast<int32_t*>(count_dst.p[owner])[src_rank * E_local + (e - owner * E_local)] = count[e];
        }
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (t >= S) return;
    uint4* rows[MAXK];
#pragma unroll
    for (int j = 0; j < MAXK; ++j) {
        rows[j] = nullptr;
        if (j < k) {
            const int slot = slot_of[(size_t)t * k + j];
            if (slot >= 0) {
                const int e = slot / cap, pos = slot - e * cap;
                const int owner = e / E_local, el = e - owner * E_local;
                // dest_filter 1: only the rows this rank keeps; 2: only the rows that go to other ranks
                const bool wanted = dest_filter == 0 || (dest_filter == 1) == (owner == src_rank);
                if (wanted && pos >= pos_lo && pos < pos_hi) {
                    const size_t row = send_base ? (size_t)el * group_rows + send_base[e] + pos
                                                 : (size_t)(src_rank * E_local + el) * cap + pos;
                    rows[j] = static_cast<uint4*>(dst.p[owner]) + row * row_vec;
                }
            }
        }
    }
    const uint4* src = x + (size_t)t * row_vec;
    for (int c = lane; c < row_vec; c += 32) {
        const uint4 v = __ldg(src + c);
#pragma unroll
        for (int j = 0; j < MAXK; ++j)
            if (rows[j]) rows[j][c] = v;
    }
}

// Valid rows of y (groups = source rank x local expert, cap rows each, count[g] valid) back to their source ranks:
// row (g, r) goes to rank g / E_local, row ((this_rank*E_local + g % E_local)*cap + r) of its buffer. A persistent
// grid walks the flattened list of valid rows (of the row window [row_lo, row_hi)) through a prefix over the counts.
__global__ void __launch_bounds__(256)
return_rows_peer_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ count, int groups, int E_local,
                        int cap, int row_vec, int this_rank, int row_lo, int row_hi, PeerPtrs dst) {
    __shared__ int s_prefix[1025];
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int running = 0;
        if (lane == 0) s_prefix[0] = 0;
        for (int g0 = 0; g0 < groups; g0 += 32) {
            const int g = g0 + lane;
            int v = g < groups ? min(max(min(count[g], cap) - row_lo, 0), row_hi - row_lo) : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, v, d);
                if (lane >= d) v += o;
            }
            if (g < groups) s_prefix[g + 1] = running + v;
            running += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int total = s_prefix[groups];
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int vrow = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; vrow < total; vrow += nwarps) {
        int lo = 0, hi = groups;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_prefix[mid] <= vrow) lo = mid; else hi = mid;
        }
        const int g = lo, r = row_lo + vrow - s_prefix[lo];
        const int owner = g / E_local, el = g - owner * E_local;
        const uint4* src = y + ((size_t)g * cap + r) * row_vec;
        uint4* out = static_cast<uint4*>(dst.p[owner]) + ((size_t)(this_rank * E_local + el) * cap + r) * row_vec;
        for (int c = lane; c < row_vec; c += 32) out[c] = __ldg(src + c);
    }
}

// From the counts of every expert at every rank (allcount[src * E + e]): where this rank's rows start inside each
// expert's dense group at the owner (send_base[e] = rows of the lower ranks), how many rows each local expert receives
// in all (dense_count[el]) and where each source's rows start in it (src_off[el * (world + 1) + s], s = 0 .. world).
__host__ __device__ inline void dense_plan_expert(const int32_t* allcount, int world, int E, int E_local, int rank, int e,
                                                  int32_t* send_base, int32_t* dense_count, int32_t* src_off) {
    int before = 0, total = 0;
    const int el = e - rank * E_local;
    const bool mine = el >= 0 && el < E_local;
    for (int s = 0; s < world; ++s) {
        if (s == rank) before = total;
        if (mine) src_off[el * (world + 1) + s] = total;
        total += allcount[s * E + e];
    }
    send_base[e] = before;
    if (mine) {
        src_off[el * (world + 1) + world] = total;
        dense_count[el] = total;
    }
}

__global__ void dense_plan_kernel(const int32_t* __restrict__ allcount, int world, int E, int E_local, int rank,
                                  int32_t* __restrict__ send_base, int32_t* __restrict__ dense_count,
                                  int32_t* __restrict__ src_off) {
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < E; e += gridDim.x * blockDim.x)
        dense_plan_expert(allcount, world, E, E_local, rank, e, send_base, dense_count, src_off);
}

}  // namespace

aristos_status_t dense_exchange_plan(const int32_t* allcount, int world, int E, int E_local, int rank,
                                     int32_t* send_base, int32_t* dense_count, int32_t* src_off, cudaStream_t st) {
    if (!allcount || !send_base || !dense_count || !src_off || world < 1 || E_local < 1 || E != world * E_local) {
        set_last_error("dense exchange plan: bad arguments");
        return ARISTOS_ERR_INVALID_ARG;
    }
    dense_plan_kernel<<<ceil_div(E, 128), 128, 0, st>>>(allcount, world, E, E_local, rank, send_base, dense_count, src_off);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

aristos_status_t permute_rows_to_peers(const void* x, const int32_t* slot_of, int S, int k, size_t row_bytes,
                                       int E_local, int cap, int src_rank, int pos_lo, int pos_hi, const PeerPtrs& dst,
                                       cudaStream_t st, const int32_t* count, int E, const PeerPtrs* count_dst,
                                       const int32_t* send_base, int group_rows, int dest_filter) {
    if (row_bytes % 16 != 0 || k > 16) { set_last_error("peer gather: row bytes must be a multiple of 16, k <= 16"); return ARISTOS_ERR_INVALID_ARG; }
    if (count && !count_dst) { set_last_error("peer gather: counts without a destination"); return ARISTOS_ERR_INVALID_ARG; }
    if (S == 0 && !count) return ARISTOS_OK;
    const int row_vec = (int)(row_bytes / 16);
    const int grid = S > 0 ? ceil_div(S, 8) : 1;
    const PeerPtrs cd = count ? *count_dst : PeerPtrs{};
    const uint4* xs = static_cast<const uint4*>(x);
    if (k <= 2) permute_rows_peer_kernel<2><<<grid, 256, 0, st>>>(xs, slot_of, S, k, row_vec, E_local, cap, src_rank, pos_lo, pos_hi, dst, count, E, cd, send_base, group_rows, dest_filter);
    else if (k <= 4) permute_rows_peer_kernel<4><<<grid, 256, 0, st>>>(xs, slot_of, S, k, row_vec, E_local, cap, src_rank, pos_lo, pos_hi, dst, count, E, cd, send_base, group_rows, dest_filter);
    else if (k <= 8) permute_rows_peer_kernel<8><<<grid, 256, 0, st>>>(xs, slot_of, S, k, row_vec, E_local, cap, src_rank, pos_lo, pos_hi, dst, count, E, cd, send_base, group_rows, dest_filter);
    else permute_rows_peer_kernel<16><<<grid, 256, 0, st>>>(xs, slot_of, S, k, row_vec, E_local, cap, src_rank, pos_lo, pos_hi, dst, count, E, cd, send_base, group_rows, dest_filter);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

aristos_status_t return_rows_to_peers(const void* y, const int32_t* count, int groups, int E_local, int cap,
                                      size_t row_bytes, int this_rank, int row_lo, int row_hi, const PeerPtrs& dst,
                                      cudaStream_t st) {
    if (row_bytes % 16 != 0 || groups > 1024) { set_last_error("peer return: bad row size or too many groups"); return ARISTOS_ERR_INVALID_ARG; }
    if (groups == 0) return ARISTOS_OK;
    return_rows_peer_kernel<<<device_sm_count() * 2, 256, 0, st>>>(static_cast<const uint4*>(y), count, groups, E_local,
                                                                   cap, (int)(row_bytes / 16), this_rank, row_lo, row_hi, dst);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace aristos

// Host-side run of the same plan (tests of the expert-parallel logic on CPU ranks).
extern "C" aristos_status_t aristos_ep_dense_plan_host(const int32_t* allcount, int world, int E, int E_local, int rank,
                                                       int32_t* send_base, int32_t* dense_count, int32_t* src_off) {
    if (!allcount || !send_base || !dense_count || !src_off || world < 1 || E_local < 1 || E != world * E_local || rank < 0 ||
        rank >= world) {
        aristos::set_last_error("dense exchange plan: bad arguments");
        return ARISTOS_ERR_INVALID_ARG;
    }
    for (int e = 0; e < E; ++e) aristos::dense_plan_expert(allcount, world, E, E_local, rank, e, send_base, dense_count, src_off);
    return ARISTOS_OK;
}
