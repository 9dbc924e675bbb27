// Expert-parallel exchange over NCCL: the library is loaded at run time (dlopen of libnccl.so.2, so a process that
// already holds NCCL - e.g. through torch - shares that copy) and only when world > 1.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <vector>

#include "../../include/aristos_moe.h"

namespace aristos {

struct EpComm;  // opaque

aristos_status_t ep_unique_id(void* out_128_bytes);
// max_ctas > 0 bounds the CTAs NCCL's kernels may use (ncclConfig_t.maxCTAs); 0 = NCCL's default.
aristos_status_t ep_comm_create(const void* unique_id_128, int rank, int world, int max_ctas, EpComm** out);
void ep_comm_destroy(EpComm* c);

// One transfer of an exchange: this rank sends `bytes` at send_offset of its send buffer to send_to and receives
// as many from recv_from into recv_offset of its receive buffer.
struct EpTransfer {
    int send_to, recv_from;
    size_t send_offset, recv_offset, bytes;
};
// Pure host logic (no CUDA, no NCCL): the transfers of one exchange, the rank's own blocks first.
std::vector<EpTransfer> ep_exchange_plan(int rank, int world, int blocks_per_peer, size_t block_stride, size_t offset,
                                         size_t len);
// Row windows of the overlapped pipeline: at most max_windows windows of a multiple of 128 rows, none smaller than
// min_rows unless the capacity itself is.
void ep_row_windows(int cap, int max_windows, int min_rows, int* window_rows, int* windows);

// All-gather of bytes_per_rank bytes (device buffers); also serves as a barrier over the ranks.
aristos_status_t ep_allgather_bytes(EpComm* c, const void* send_dev, void* recv_dev, size_t bytes_per_rank,
                                    cudaStream_t stream);

// One grouped exchange. For every peer d != rank and every block b < blocks_per_peer:
//   send  bytes [ (d*blocks_per_peer + b) * block_stride + offset, +len )  of send_buf to d
//   recv  bytes [ (d*blocks_per_peer + b) * block_stride + offset, +len )  of recv_buf from d
// The rank's own blocks are copied device-to-device on the same stream.
aristos_status_t ep_all_to_all_blocks(EpComm* c, const void* send_buf, void* recv_buf, int blocks_per_peer,
                                      size_t block_stride, size_t offset, size_t len, cudaStream_t stream);

}  // namespace aristos
