// Expert-parallel exchange over peer memory: one exchange region per rank (flag words | received counts | received
// rows | returned outputs | scales), mapped into every other rank through CUDA IPC. Rows reach it either by kernels
// that store through the peer mappings (the gather kernel of ep_kernels.cu, the expert GEMM's output tiles) or by the
// copy engines (cudaMemcpy2DAsync of row windows); arrival is published by a one-warp kernel that stores an epoch
// number into the destination's flag word, and consumers order their streams behind those flags with stream memory
// operations (cuStreamWaitValue32). No kernel spins on a peer.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/aristos_moe.h"
#include "ep_nccl.h"

namespace aristos {

struct EpP2P;

enum { EP_FLAG_IN = 0, EP_FLAG_RET = 1, EP_FLAG_COUNT = 2 };
constexpr int EP_MAX_WINDOWS = 16;

// Collective over the ranks of `bootstrap` (used for the IPC-handle exchange and as a start barrier). The exchange
// region holds, per rank: flag words, the received row counts (groups int32), xr (xr_bytes) and yg (yg_bytes).
// Returns ARISTOS_ERR_UNSUPPORTED on EVERY rank when any rank could not allocate or map (all ranks then choose the
// same fallback); other errors mean the bootstrap collective itself failed.
aristos_status_t ep_p2p_create(EpComm* bootstrap, int rank, int world, int groups, size_t xr_bytes, size_t yg_bytes,
                               size_t aux_bytes, EpP2P** out);
void ep_p2p_destroy(EpP2P* p);
// The transport decision every rank takes from the all-gathered per-rank flags: peer memory only if it works on all.
bool ep_transport_agreed(const int* ok_flags, int world);
void* ep_p2p_xr(EpP2P* p);
void* ep_p2p_yg(EpP2P* p);
void* ep_p2p_aux(EpP2P* p);   // third exchange buffer (the fp8 path keeps the received activation scales there)
// Every rank's copy of one exchange buffer as mapped into this process (out[world]); kernels store through them.
enum { EP_BUF_XR = 0, EP_BUF_YG = 1, EP_BUF_AUX = 2, EP_BUF_RCOUNT = 3 };
constexpr int EP_MAX_RANKS = 16;
void ep_p2p_peer_ptrs(EpP2P* p, int which, void** out);
int32_t* ep_p2p_rcount(EpP2P* p);
// Starts a new forward: every flag of this forward is compared against the returned epoch.
uint32_t ep_p2p_begin(EpP2P* p);
// Push block b of peer d (b < blocks_per_peer) of send_buf to block (rank*blocks_per_peer + b) of the destination's
// buffer `which` (EP_FLAG_IN: xr, EP_FLAG_RET: yg, EP_FLAG_COUNT: rcount), bytes [offset, offset + len) of each block.
aristos_status_t ep_p2p_push(EpP2P* p, int which, const void* send_buf, int blocks_per_peer, size_t block_stride,
                             size_t offset, size_t len, cudaStream_t stream);
// After the pushes of (kind, window) on the same stream: publish them to every rank.
aristos_status_t ep_p2p_signal(EpP2P* p, int kind, int window, cudaStream_t stream);
// Order `stream` behind the arrival of (kind, window) from every rank.
aristos_status_t ep_p2p_wait(EpP2P* p, int kind, int window, cudaStream_t stream);
// This rank's flag words of (kind, window), indexed by source rank, and the epoch of the current forward: what a
// kernel needs to wait for one source's rows itself instead of ordering the whole stream behind every rank.
const uint32_t* ep_p2p_flags(const EpP2P* p, int kind, int window);
uint32_t ep_p2p_epoch(const EpP2P* p);
// One small kernel: count[e] of every expert goes into its owner's received-count list (entry rank * E_local +
// e % E_local) and the EP_FLAG_COUNT flag (window 0) of this rank is raised at every rank.
// With to_all every rank also receives the whole list in its all-counts table (ep_p2p_allcount: entry src * E + e).
aristos_status_t ep_p2p_send_counts(EpP2P* p, const int32_t* count, int E, int E_local, cudaStream_t stream,
                                    bool to_all = false);
int32_t* ep_p2p_allcount(EpP2P* p);
// The flag page as plain words (host-side mirror of what the kernels and stream waits do; used by the release below
// and by tests that run the protocol among CPU ranks).
int ep_flag_words();
int ep_flag_word_index(int kind, int window, int src);
uint32_t ep_flags_pending(const uint32_t* words, uint32_t epoch, int world, int kind, int window);
void ep_flags_release(uint32_t* words, uint32_t epoch);
// Host-side release: store the current epoch into every one of THIS rank's flag words, so that stream waits and
// kernel waits of the current forward that a missing peer left unsatisfied complete (their data is then undefined;
// the caller marks the forward failed).
aristos_status_t ep_p2p_release_local_waits(EpP2P* p);

}  // namespace aristos
