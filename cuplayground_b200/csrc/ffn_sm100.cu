// Expert FFN on the 5th-generation tensor cores: a persistent, warp-specialised grouped GEMM.
//
// Replaces, for bf16, fp16 and tf32 (fp32 storage), the reference's fused expert tile fGET / deviceCollectiveMMA (mma.cuh:46-179, :198-369: one
// CTA per 128x64 tile, CUTLASS sm80 cp.async mainloop, mma.sync, accumulators transposed through shared memory,
// epilogue act(acc + bias) from processor/tiling.cuh:29-57) and its software tile schedulers sK / wScheduler
// (auditorium/scheduling.cuh:202-265, warpScheduler.cuh:267-344: doorbells and ready queues in global memory that
// hand GEMM0 / GEMM1 tile ids to persistent "processor" CTAs).
//
// One launch computes  out[g, r, n0:n0+W] = epi( A[g, r, :] * B[expert(g), n, :]^T )  for every row group g:
//   up-projection   : A = gathered tokens (groups, rows, H), B = W1 (and W3), out = h, epi = relu | gelu | swiglu
//   down-projection : A = h (groups, rows, I),               B = W2,          out = y, epi = identity
// Operands are (rows, K) row-major = K-major, the reference's A (M,K) / B (N,K) convention (mma.cuh:394-397).
//
// Per CTA (one per SM, 192 threads):
//   warp 0    TMA producer: 3-D tiled loads (K, rows, group) of a 128x64 A box and two 128x64 B boxes per stage
//             into 128-byte-swizzled shared memory, completion on an mbarrier
//   warp 1    MMA issuer: one thread issues tcgen05.mma (M128 x N256 x K16, bf16 -> fp32) into one of two
//             256-column TMEM accumulators; tcgen05.commit releases the stage / publishes the accumulator
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its 32-lane quarter), activation, bf16, 16-byte
//             stores masked by the group's row count; runs under the next tile's main loop
// SwiGLU puts W1 rows in B rows 0-127 and W3 rows in B rows 128-255 of the same MMA, so gate and up share one pass
// over A and the epilogue multiplies silu(acc[:, c]) * acc[:, 128 + c].
// Tile schedule: every CTA builds the same prefix over groups of (valid 128-row tiles x column tiles) from the
// device-resident counts and walks tiles blockIdx, blockIdx + grid, ... (row tile fastest, so concurrently running
// CTAs share B panels through L2). Nothing is read back to the host and empty tiles cost nothing.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "ffn_internal.h"
#include "ptx_sm100.cuh"
#include "tensor_map.cuh"

namespace aristos {

namespace {

constexpr int BM = 128;          // rows per tile
constexpr int BN = 256;          // MMA N (B rows per stage)
constexpr int BK = 64;           // K per stage (128 bytes of bf16 = one swizzle row)
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_HALF_BYTES = 128 * BK * 2;
constexpr int B_STAGE_BYTES = 2 * B_HALF_BYTES;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int FFN_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int TMEM_COLS = 512;   // two 256-column accumulators
constexpr int MAX_GROUPS = 1024;
constexpr int SMEM_AUX_BYTES = 256 + (MAX_GROUPS + 1) * 4;
constexpr int STAGING_BYTES = 128 * 128;   // 128 rows x 64 bf16 of epilogue output, 128-byte swizzled
constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * STAGE_BYTES + STAGING_BYTES + SMEM_AUX_BYTES;

enum { FMT_BF16 = 0, FMT_F16 = 1, FMT_TF32 = 2 };

struct FfnGemmParams {
    const int32_t* count;   // valid rows per group
    int groups;
    int experts;            // expert of group g = g % experts
    int rows_per_group;
    int row_begin, row_end; // row window inside every group
    int N;                  // output columns
    int K;
    int gated;              // 1: B half 1 comes from the second weight tensor at the same rows (SwiGLU)
    int act;                // ARISTOS_ACT_* for the non-gated epilogue
    void* out;              // (groups * rows_per_group, N), 16-bit elements
    int self_source;        // expert parallel: rows of this source rank need no arrival flag (gathered on the launching
                            // stream); -1: none. (The struct is kept at 128 bytes: one more member changes how the
                            // compiler treats the kernel argument and cost the small-K configurations 30 %.)
    const void* bias0;      // (experts, N) added to the accumulator before the activation, or nullptr
    const void* bias1;      // SwiGLU: bias of the second (up) projection, or nullptr
    int32_t* dev_status;
    int peer_world;         // > 0: output tiles go straight to the rank that sent the rows (group g came from rank
    int peer_rank;          //      g / experts) through PeerOutMaps, as group peer_rank * experts + g % experts
    int rows_mode;          // ROWS_ALL, ROWS_FULL_PAIRS (pair kernel: whole 256-row tiles only) or ROWS_TAIL (single-CTA
                            // kernel: the < 256 rows per group that the pair kernel left)
    int band;               // row tiles per band of the tile order (band_tile_coord); 0 = row tile fastest
    int first_source;       // ring start of the source order inside an expert (this rank: its own rows come first)
    // Arrival flags of the rows of each source rank (expert parallel, rows stored by the peers' gather kernels):
    // the producer waits until src_flags[src] has reached flag_epoch before it loads the first tile of a group that
    // came from rank src. nullptr: the rows are complete before the launch.
    const uint32_t* src_flags;
    uint32_t flag_epoch;
    uint32_t flag_limit_ms;
};
static_assert(sizeof(FfnGemmParams) == 128, "FfnGemmParams: keep the kernel argument at 128 bytes");

enum { ROWS_ALL = 0, ROWS_FULL_PAIRS = 1, ROWS_TAIL = 2 };

// One output tensor map per source rank: that rank's buffer for returned expert outputs, (all experts, rows, N),
// mapped into this process. The epilogue's TMA store then IS the return all-to-all, tile by tile.
constexpr int MAX_PEER_OUT = 8;
struct PeerOutMaps {
    CUtensorMap m[MAX_PEER_OUT];
    void* base[MAX_PEER_OUT];
};
// Kernel argument: the maps for the instantiations that return tiles to peers, one word for those that do not (the
// kernels are specialised on the operand format, on bias and on peer output at compile time, so the common case -
// bf16, no bias, local output - carries none of the other cases' instructions, registers or arguments).
template <bool PEERS>
struct PeerMapsArg {
    CUtensorMap m[MAX_PEER_OUT];
    void* base[MAX_PEER_OUT];     // the same buffers as raw pointers (row-masked stores of partly valid tiles), or null
};
template <>
struct PeerMapsArg<false> {
    int unused;
};

// Rows of group g inside the row window of this launch.
__device__ __forceinline__ int window_rows(const FfnGemmParams& p, int g) {
    return max(0, min(p.count[g] - p.row_begin, p.row_end - p.row_begin));
}
// Row tiles this launch computes for a group with `rows` rows in the window (TILE_ROWS = 128 or 256).
template <int TILE_ROWS>
__device__ __forceinline__ int row_tiles_of(const FfnGemmParams& p, int rows) {
    if (p.rows_mode == ROWS_FULL_PAIRS) return rows / 256;
    if (p.rows_mode == ROWS_TAIL) return (rows % 256 + 127) / 128;
    return (rows + TILE_ROWS - 1) / TILE_ROWS;
}
struct TileCoord {
    int g, m0, n0;
};
// Tile number -> (group, first row, first output column); vg walks forward through the prefix.
template <int TILE_ROWS>
__device__ __forceinline__ TileCoord decode_tile(const FfnGemmParams& p, const int* prefix, int& vg, int tile,
                                                 int n_tiles, int out_w) {
    while (tile >= prefix[vg + 1]) ++vg;
    TileCoord t;
    t.g = ordered_group(vg, p.groups, p.experts, p.first_source);
    const int local = tile - prefix[vg];
    const int mt = (prefix[vg + 1] - prefix[vg]) / n_tiles;
    int m, n;
    band_tile_coord(local, mt, n_tiles, p.band, &m, &n);
    const int start = p.rows_mode == ROWS_TAIL ? (window_rows(p, t.g) / 256) * 256 : 0;
    t.m0 = p.row_begin + start + m * TILE_ROWS;
    t.n0 = n * out_w;
    return t;
}
// Every CTA builds the same prefix over the groups (in walking order) of tiles per group; one warp, 32 groups a step.
template <int TILE_ROWS>
__device__ __forceinline__ void build_tile_prefix(const FfnGemmParams& p, int* prefix, int n_tiles, int lane) {
    int running = 0;
    if (lane == 0) prefix[0] = 0;
    for (int g0 = 0; g0 < p.groups; g0 += 32) {
        const int g = g0 + lane;
        int v = 0;
        if (g < p.groups)
            v = row_tiles_of<TILE_ROWS>(p, window_rows(p, ordered_group(g, p.groups, p.experts, p.first_source))) * n_tiles;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += o;
        }
        if (g < p.groups) prefix[g + 1] = running + v;
        running += __shfl_sync(0xffffffffu, v, 31);
    }
}
// Producer side of the device-initiated exchange (the reference's nvshmem_signal_wait_until before each peer's GEMM,
// auditorium/overlap.cuh:102-105, with a limit): before the first load of rows that came from rank src, wait until
// that rank's arrival flag has reached this forward's epoch. `seen` caches the sources already observed.
__device__ __forceinline__ bool wait_source_rows(const FfnGemmParams& p, int g, uint32_t& seen, volatile int* abort_flag) {
    if (p.src_flags == nullptr) return true;
    const int src = g / p.experts;
    if (src == p.self_source || ((seen >> src) & 1u)) return true;
    if (!ptx::flag_wait_bounded(p.src_flags + src, p.flag_epoch, abort_flag, p.dev_status,
                                (uint64_t)p.flag_limit_ms * 1000000ull))
        return false;
    seen |= 1u << src;
    return true;
}

// The first `valid` rows of the 128 x 128-byte swizzled staging tile to global memory (row pitch `pitch` bytes), by
// the 128 epilogue threads: 8 threads per row, 16 rows per step, 16-byte stores that together fill whole 128-byte lines.
__device__ __forceinline__ void copy_valid_rows(uint32_t staging, uint8_t* dst, size_t pitch, int valid, int epi_tid) {
    const int ch = epi_tid & 7;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int r = it * 16 + (epi_tid >> 3);
        if (r < valid) {
            uint4 v;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(staging + r * 128 + ((ch ^ (r & 7)) << 4)));
            *reinterpret_cast<uint4*>(dst + (size_t)r * pitch + ch * 16) = v;
        }
    }
}

// Destination of a partly valid 128-row tile whose output goes to rank src: row m0 of group og in that rank's buffer,
// or nullptr for a whole tile (which leaves by TMA store). Partly valid tiles are stored row by row, valid rows only.
template <int FMT>
__device__ __forceinline__ uint8_t* masked_peer_rows(const FfnGemmParams& p, void* base, int og, int g, int m0, int rows) {
    const int row_limit = min(p.count[g], p.row_end);
    if (base == nullptr || m0 >= row_limit || m0 + rows <= row_limit) return nullptr;
    constexpr size_t elt = FMT == FMT_TF32 ? 4 : 2;
    return static_cast<uint8_t*>(base) + ((size_t)og * p.rows_per_group + m0) * p.N * elt;
}

__device__ __forceinline__ uint32_t pack_16bit(float a, float b, int fmt) {
    if (fmt == FMT_F16) {
        __half2 t = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&t);
    }
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
}

// acc[0..31] += bias[0..31] (the same bytes for every thread of the CTA: a broadcast load).
__device__ __forceinline__ void add_bias32(uint32_t (&acc)[32], const void* bias, size_t elem_offset, int fmt) {
    if (fmt == FMT_TF32) {
        const float4* b = reinterpret_cast<const float4*>(static_cast<const float*>(bias) + elem_offset);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 v = __ldg(b + q);
            acc[4 * q] = __float_as_uint(__uint_as_float(acc[4 * q]) + v.x);
            acc[4 * q + 1] = __float_as_uint(__uint_as_float(acc[4 * q + 1]) + v.y);
            acc[4 * q + 2] = __float_as_uint(__uint_as_float(acc[4 * q + 2]) + v.z);
            acc[4 * q + 3] = __float_as_uint(__uint_as_float(acc[4 * q + 3]) + v.w);
        }
        return;
    }
    const uint4* b = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(bias) + elem_offset);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint4 u = __ldg(b + q);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            if (fmt == FMT_F16) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                lo = f.x; hi = f.y;
            } else {
                lo = __uint_as_float(w[i] << 16);
                hi = __uint_as_float(w[i] & 0xFFFF0000u);
            }
            acc[q * 8 + 2 * i] = __float_as_uint(__uint_as_float(acc[q * 8 + 2 * i]) + lo);
            acc[q * 8 + 2 * i + 1] = __float_as_uint(__uint_as_float(acc[q * 8 + 2 * i + 1]) + hi);
        }
    }
}

// Epilogue of one 128-row tile, run by the four epilogue warps of a CTA (thread = accumulator row): TMEM -> registers
// -> activation -> bf16 -> 128-byte-swizzled shared staging (64 output columns at a time) -> TMA store. The
// accumulator buffer is handed back as soon as the last TMEM load has landed. A tile that lies entirely at or past
// the group's valid rows stores nothing; a partly valid tile stores all of its 128 rows (the extra rows hold
// unspecified values, never past the group's row capacity: the tensor map clips them). With masked_dst != nullptr
// (a partly valid tile whose rows go to another rank: masked_dst = row m0 of the destination group there) every thread
// stores its own row with 16-byte stores if the row is valid, so that only rows that exist cross NVLink.
template <bool PAIR, int FMT, bool BIAS, bool MASKABLE>
__device__ __forceinline__ void epilogue_tile(const FfnGemmParams& p, const CUtensorMap* tmOut, int out_g, int g, int m0,
                                              int n0, int row_in_tile, uint32_t taddr, uint32_t tempty, int lane,
                                              int epi_tid, uint32_t staging, uint8_t* masked_dst = nullptr) {
    const int row_limit = min(p.count[g], p.row_end);
    const bool tile_live = m0 < row_limit;
    const bool masked = MASKABLE && masked_dst != nullptr;       // the same for all epilogue threads of the tile
    const int nchunk = p.gated ? 2 : 4;              // 64-column chunks of the output tile
    const uint32_t my_row = staging + row_in_tile * 128;
    const int sw = row_in_tile & 7;
#pragma unroll 1
    for (int c = 0; c < nchunk; ++c) {
        if (epi_tid == 0) ptx::bulk_wait_group_read0();      // the previous store has drained the staging buffer
        ptx::named_barrier_sync(1, EPI_THREADS);
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
            const int col = c * 64 + hlf * 32;
            uint32_t a[32], b[32];
            ptx::tmem_ld_32x32b_x32(taddr + col, a);
            if (p.gated) ptx::tmem_ld_32x32b_x32(taddr + 128 + col, b);
            ptx::tmem_ld_wait();
            if (c == nchunk - 1 && hlf == 1) {
                ptx::tcgen05_fence_before();
                if (PAIR) {
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_cluster(tempty);
                } else {
                    ptx::mbar_arrive(tempty);
                }
            }
            if (BIAS && n0 + col < p.N) {  // act(acc + bias), the reference's epilogue (processor/tiling.cuh:29-57)
                const size_t boff = (size_t)(g % p.experts) * p.N + n0 + col;
                if (p.bias0) add_bias32(a, p.bias0, boff, FMT);
                if (p.gated && p.bias1) add_bias32(b, p.bias1, boff, FMT);
            }
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float v0 = __uint_as_float(a[2 * i]), v1 = __uint_as_float(a[2 * i + 1]);
                if (p.gated) {
                    v0 = act_silu(v0) * __uint_as_float(b[2 * i]);
                    v1 = act_silu(v1) * __uint_as_float(b[2 * i + 1]);
                } else if (p.act == ARISTOS_ACT_RELU) { v0 = act_relu(v0); v1 = act_relu(v1); }
                else if (p.act == ARISTOS_ACT_GELU) { v0 = act_gelu(v0); v1 = act_gelu(v1); }
                o[i] = pack_16bit(v0, v1, FMT);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = hlf * 4 + i;               // 16-byte chunk of the 128-byte staging row
                ptx::st_shared_v4(my_row + ((j ^ sw) << 4), o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
        }
        ptx::fence_proxy_async_shared();
        ptx::named_barrier_sync(1, EPI_THREADS);
        if (MASKABLE && masked) {
            // the valid rows only, 8 threads per 128-byte row: whole lines leave for the other rank
            if (n0 + c * 64 < p.N) copy_valid_rows(staging, masked_dst + (size_t)(n0 + c * 64) * 2, (size_t)p.N * 2,
                                                   row_limit - m0, epi_tid);
        } else if (epi_tid == 0 && tile_live && n0 + c * 64 < p.N) {
            ptx::tma_store_3d(tmOut, staging, n0 + c * 64, m0, out_g);
            ptx::bulk_commit_group();
        }
    }
}

// The same for fp32 output (tf32 path): a 128-byte staging row holds 32 columns, so the tile leaves in 32-column
// chunks.
template <bool PAIR, bool BIAS, bool MASKABLE>
__device__ __forceinline__ void epilogue_tile_f32(const FfnGemmParams& p, const CUtensorMap* tmOut, int out_g, int g,
                                                  int m0, int n0, int row_in_tile, uint32_t taddr, uint32_t tempty,
                                                  int lane, int epi_tid, uint32_t staging, uint8_t* masked_dst = nullptr) {
    const int row_limit = min(p.count[g], p.row_end);
    const bool tile_live = m0 < row_limit;
    const bool masked = MASKABLE && masked_dst != nullptr;
    const int nchunk = p.gated ? 4 : 8;
    const uint32_t my_row = staging + row_in_tile * 128;
    const int sw = row_in_tile & 7;
#pragma unroll 1
    for (int c = 0; c < nchunk; ++c) {
        if (epi_tid == 0) ptx::bulk_wait_group_read0();
        ptx::named_barrier_sync(1, EPI_THREADS);
        const int col = c * 32;
        uint32_t a[32], b[32];
        ptx::tmem_ld_32x32b_x32(taddr + col, a);
        if (p.gated) ptx::tmem_ld_32x32b_x32(taddr + 128 + col, b);
        ptx::tmem_ld_wait();
        if (c == nchunk - 1) {
            ptx::tcgen05_fence_before();
            if (PAIR) {
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(tempty);
            } else {
                ptx::mbar_arrive(tempty);
            }
        }
        if (BIAS && n0 + col < p.N) {
            const size_t boff = (size_t)(g % p.experts) * p.N + n0 + col;
            if (p.bias0) add_bias32(a, p.bias0, boff, FMT_TF32);
            if (p.gated && p.bias1) add_bias32(b, p.bias1, boff, FMT_TF32);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(a[i]);
            if (p.gated) v = act_silu(v) * __uint_as_float(b[i]);
            else if (p.act == ARISTOS_ACT_RELU) v = act_relu(v);
            else if (p.act == ARISTOS_ACT_GELU) v = act_gelu(v);
            a[i] = __float_as_uint(v);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            ptx::st_shared_v4(my_row + ((j ^ sw) << 4), a[4 * j], a[4 * j + 1], a[4 * j + 2], a[4 * j + 3]);
        ptx::fence_proxy_async_shared();
        ptx::named_barrier_sync(1, EPI_THREADS);
        if (MASKABLE && masked) {
            if (n0 + col < p.N) copy_valid_rows(staging, masked_dst + (size_t)(n0 + col) * 4, (size_t)p.N * 4, row_limit - m0,
                                                epi_tid);
        } else if (epi_tid == 0 && tile_live && n0 + col < p.N) {
            ptx::tma_store_3d(tmOut, staging, n0 + col, m0, out_g);
            ptx::bulk_commit_group();
        }
    }
}

template <int FMT, bool BIAS, bool PEERS>
__global__ void __launch_bounds__(FFN_THREADS, 1)
ffn_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                        const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmOut,
                        const __grid_constant__ PeerMapsArg<PEERS> peers, const FfnGemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t staging = ptx::smem_u32(smem + STAGES * STAGE_BYTES);
    uint8_t* aux = smem + STAGES * STAGE_BYTES + STAGING_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aux);             // full[S], empty[S], tfull[2], tempty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 132);
    int* prefix = reinterpret_cast<int*>(aux + 256);               // [groups + 1] tiles before group g

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t smem_base = ptx::smem_u32(smem);

    const int out_w = p.gated ? 128 : 256;             // output columns per tile
    const int n_tiles = (p.N + out_w - 1) / out_w;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, EPI_THREADS);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        build_tile_prefix<BM>(p, prefix, n_tiles, lane);
    } else if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[p.groups];
    constexpr int bke = FMT == FMT_TF32 ? BK / 2 : BK;   // elements of K per stage: 128 bytes
    const int kblocks = p.K / bke;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB0);
            ptx::prefetch_tensormap(&tmB1);
            int stage = 0;
            uint32_t phase = 0;
            int vg = 0;
            uint32_t seen = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileCoord t = decode_tile<BM>(p, prefix, vg, tile, n_tiles, out_w);
                const int g = t.g, m0 = t.m0, n0 = t.n0;
                const int e = g % p.experts;
                const int n1 = p.gated ? n0 : n0 + 128;
                ok = wait_source_rows(p, g, seen, abort_flag);
                if (!ok) break;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.dev_status);
                    if (!ok) break;
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(full, STAGE_BYTES);
                    ptx::tma_load_3d(sa, &tmA, kb * bke, m0, g, full);
                    ptx::tma_load_3d(sa + A_STAGE_BYTES, &tmB0, kb * bke, n0, e, full);
                    ptx::tma_load_3d(sa + A_STAGE_BYTES + B_HALF_BYTES, &tmB1, kb * bke, n1, e, full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc_f32acc(BM, BN, FMT == FMT_BF16 ? 1u : (FMT == FMT_F16 ? 0u : 2u));
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ok = ptx::mbar_wait_bounded(bar_tempty + 8 * buf, aphase ^ 1u, abort_flag, p.dev_status);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_full + 8 * stage, phase, abort_flag, p.dev_status);
                    if (!ok) break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    const uint64_t da = ptx::umma_desc_k_sw128(sa);
                    const uint64_t db = ptx::umma_desc_k_sw128(sa + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advance 32 bytes (16 bf16) along K inside the swizzled row: +2 in 16-byte units
                        if constexpr (FMT == FMT_TF32) ptx::umma_tf32(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else ptx::umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(bar_tfull + 8 * buf);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;                 // TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        const int epi_tid = threadIdx.x - 64;
        int vg = 0;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileCoord t = decode_tile<BM>(p, prefix, vg, tile, n_tiles, out_w);
            const int g = t.g, m0 = t.m0, n0 = t.n0;
            const int buf = it & 1;
            const uint32_t aphase = (it >> 1) & 1u;
            ok = ptx::mbar_wait_bounded(bar_tfull + 8 * buf, aphase, abort_flag, p.dev_status);
            // the tile's epilogue synchronises the four warps: they must agree on leaving
            ok = !ptx::named_barrier_or(2, EPI_THREADS, !ok);
            if (!ok) break;
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const CUtensorMap* om = &tmOut;
            int og = g;
            uint8_t* md = nullptr;
            if constexpr (PEERS) {
                const int src = g / p.experts;
                om = &peers.m[src];
                og = p.peer_rank * p.experts + (g - src * p.experts);
                md = masked_peer_rows<FMT>(p, peers.base[src], og, g, m0, BM);
            }
            if constexpr (FMT == FMT_TF32)
                epilogue_tile_f32<false, BIAS, PEERS>(p, om, og, g, m0, n0, row_in_tile, taddr, bar_tempty + 8 * buf, lane, epi_tid, staging, md);
            else
                epilogue_tile<false, FMT, BIAS, PEERS>(p, om, og, g, m0, n0, row_in_tile, taddr, bar_tempty + 8 * buf, lane, epi_tid, staging, md);
        }
        if (epi_tid == 0) ptx::bulk_wait_group0();
    }

    ptx::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- up and down projection in one persistent launch ------------------------------------------------------------------
// For small row groups (many experts, a few row tiles each) the two projections of a layer are one launch: the tile list
// is every up-projection tile followed by every down-projection tile, and a down tile of (group, row tile) becomes
// ready when all the up-projection column tiles of that row tile have stored their part of h - the dependency the
// reference's schedulers model with per-row-tile queues of second-GEMM tasks (auditorium/scheduling.cuh:212-216,
// warpScheduler.cuh:280-285: "sTB" tasks appear when a row of "fTB" tiles is complete). Here the epilogue of an up tile
// counts itself into done[group][row tile] once its TMA stores have completed, and the producer of a down tile waits
// (bounded) until the count has reached the number of up column tiles. Every CTA walks its tiles in order and all up
// tiles precede all down tiles, so no up tile ever waits behind a down tile: the wait cannot deadlock. There is no
// drain between the projections, the tail of the up projection overlaps the head of the down projection, and h is
// read back while it is still in L2.
__device__ __forceinline__ TileCoord decode_phase_tile(const FfnGemmParams& p, const int* rt_prefix, int& vg, int t,
                                                       int n_tiles, int out_w) {
    // t counts the tiles of one projection: groups in walking order, inside a group the row tile runs fastest
    while (t >= rt_prefix[vg + 1] * n_tiles) ++vg;
    TileCoord c;
    c.g = ordered_group(vg, p.groups, p.experts, p.first_source);
    const int local = t - rt_prefix[vg] * n_tiles;
    const int mt = rt_prefix[vg + 1] - rt_prefix[vg];
    c.m0 = p.row_begin + (local % mt) * BM;
    c.n0 = (local / mt) * out_w;
    return c;
}

template <int FMT, bool BIAS, bool PEERS>
__global__ void __launch_bounds__(FFN_THREADS, 1)
ffn_updown_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB00,
                  const __grid_constant__ CUtensorMap tmB01, const __grid_constant__ CUtensorMap tmOut0,
                  const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                  const __grid_constant__ CUtensorMap tmOut1, const __grid_constant__ PeerMapsArg<PEERS> peers,
                  const FfnGemmParams p0, const FfnGemmParams p1, int32_t* __restrict__ done, int max_row_tiles) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t staging = ptx::smem_u32(smem + STAGES * STAGE_BYTES);
    uint8_t* aux = smem + STAGES * STAGE_BYTES + STAGING_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aux);             // full[S], empty[S], tfull[2], tempty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 132);
    int* rt_prefix = reinterpret_cast<int*>(aux + 256);            // [groups + 1] row tiles before group g

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t smem_base = ptx::smem_u32(smem);

    const int out_w0 = p0.gated ? 128 : 256;
    const int nt0 = (p0.N + out_w0 - 1) / out_w0;
    const int nt1 = (p1.N + 255) / 256;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, EPI_THREADS);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        build_tile_prefix<BM>(p0, rt_prefix, 1, lane);          // n_tiles = 1: a prefix over row tiles
    } else if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int row_tiles = rt_prefix[p0.groups];
    const int T0 = row_tiles * nt0, total_tiles = T0 + row_tiles * nt1;
    constexpr int bke = FMT == FMT_TF32 ? BK / 2 : BK;
    const int kblocks0 = p0.K / bke, kblocks1 = p1.K / bke;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmA0);
            ptx::prefetch_tensormap(&tmB00);
            ptx::prefetch_tensormap(&tmB01);
            ptx::prefetch_tensormap(&tmA1);
            ptx::prefetch_tensormap(&tmB1);
            int stage = 0;
            uint32_t phase = 0;
            int vg0 = 0, vg1 = 0;
            uint32_t seen = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const bool down = tile >= T0;
                const TileCoord t = down ? decode_phase_tile(p1, rt_prefix, vg1, tile - T0, nt1, 256)
                                         : decode_phase_tile(p0, rt_prefix, vg0, tile, nt0, out_w0);
                const int g = t.g, m0 = t.m0, n0 = t.n0;
                const int e = g % p0.experts;
                const CUtensorMap *mA, *mB0, *mB1;
                int n1, kblocks;
                if (down) {
                    // every up-projection column tile of this row tile must have stored its part of h
                    const int rt = (m0 - p1.row_begin) / BM;
                    ok = ptx::flag_wait_bounded(reinterpret_cast<const uint32_t*>(done + g * max_row_tiles + rt),
                                                (uint32_t)nt0, abort_flag, p1.dev_status);
                    if (!ok) break;
                    mA = &tmA1; mB0 = &tmB1; mB1 = &tmB1; n1 = n0 + 128; kblocks = kblocks1;
                } else {
                    ok = wait_source_rows(p0, g, seen, abort_flag);
                    if (!ok) break;
                    mA = &tmA0; mB0 = &tmB00; mB1 = &tmB01; n1 = p0.gated ? n0 : n0 + 128; kblocks = kblocks0;
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p0.dev_status);
                    if (!ok) break;
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(full, STAGE_BYTES);
                    ptx::tma_load_3d(sa, mA, kb * bke, m0, g, full);
                    ptx::tma_load_3d(sa + A_STAGE_BYTES, mB0, kb * bke, n0, e, full);
                    ptx::tma_load_3d(sa + A_STAGE_BYTES + B_HALF_BYTES, mB1, kb * bke, n1, e, full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc_f32acc(BM, BN, FMT == FMT_BF16 ? 1u : (FMT == FMT_F16 ? 0u : 2u));
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const int kblocks = tile >= T0 ? kblocks1 : kblocks0;
                const int buf = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ok = ptx::mbar_wait_bounded(bar_tempty + 8 * buf, aphase ^ 1u, abort_flag, p0.dev_status);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_full + 8 * stage, phase, abort_flag, p0.dev_status);
                    if (!ok) break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    const uint64_t da = ptx::umma_desc_k_sw128(sa);
                    const uint64_t db = ptx::umma_desc_k_sw128(sa + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        if constexpr (FMT == FMT_TF32) ptx::umma_tf32(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else ptx::umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(bar_tfull + 8 * buf);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const int epi_tid = threadIdx.x - 64;
        int vg0 = 0, vg1 = 0;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const bool down = tile >= T0;
            const TileCoord t = down ? decode_phase_tile(p1, rt_prefix, vg1, tile - T0, nt1, 256)
                                     : decode_phase_tile(p0, rt_prefix, vg0, tile, nt0, out_w0);
            const int g = t.g, m0 = t.m0, n0 = t.n0;
            const int buf = it & 1;
            const uint32_t aphase = (it >> 1) & 1u;
            ok = ptx::mbar_wait_bounded(bar_tfull + 8 * buf, aphase, abort_flag, p0.dev_status);
            ok = !ptx::named_barrier_or(2, EPI_THREADS, !ok);
            if (!ok) break;
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            if (!down) {
                if constexpr (FMT == FMT_TF32)
                    epilogue_tile_f32<false, BIAS, false>(p0, &tmOut0, g, g, m0, n0, row_in_tile, taddr, bar_tempty + 8 * buf, lane, epi_tid, staging);
                else
                    epilogue_tile<false, FMT, BIAS, false>(p0, &tmOut0, g, g, m0, n0, row_in_tile, taddr, bar_tempty + 8 * buf, lane, epi_tid, staging);
                // this tile's part of h is complete in global memory: count it for the down projection's producers
                if (epi_tid == 0) {
                    ptx::bulk_wait_group0();
                    asm volatile("fence.proxy.async;" ::: "memory");
                    __threadfence();
                    atomicAdd(done + g * max_row_tiles + (m0 - p0.row_begin) / BM, 1);
                }
            } else {
                const CUtensorMap* om = &tmOut1;
                int og = g;
                uint8_t* md = nullptr;
                if constexpr (PEERS) {
                    const int src = g / p1.experts;
                    om = &peers.m[src];
                    og = p1.peer_rank * p1.experts + (g - src * p1.experts);
                    md = masked_peer_rows<FMT>(p1, peers.base[src], og, g, m0, BM);
                }
                if constexpr (FMT == FMT_TF32)
                    epilogue_tile_f32<false, BIAS, PEERS>(p1, om, og, g, m0, n0, row_in_tile, taddr, bar_tempty + 8 * buf, lane, epi_tid, staging, md);
                else
                    epilogue_tile<false, FMT, BIAS, PEERS>(p1, om, og, g, m0, n0, row_in_tile, taddr, bar_tempty + 8 * buf, lane, epi_tid, staging, md);
            }
        }
        if (epi_tid == 0) ptx::bulk_wait_group0();
    }

    ptx::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- CTA-pair variant --------------------------------------------------------------------------------------------------
// Two CTAs on the two SMs of a TPC work on one 256 x 256 tile with tcgen05 cta_group::2: each CTA stages its own 128
// rows of A and its own 128 rows of B (for SwiGLU: CTA 0 the W1 rows, CTA 1 the W3 rows), the first CTA's MMA thread
// issues M256 x N256 x K16 instructions that read both CTAs' shared memory, and each CTA's TMEM receives its 128 rows
// of the accumulator. Per SM that halves the B bytes staged and read per FLOP (32 KB instead of 48 KB per stage,
// six stages instead of four). Used when the row groups are large; small groups keep the single-CTA tiles.
constexpr int P_STAGES = 6;
constexpr int P_STAGE_BYTES = A_STAGE_BYTES + B_HALF_BYTES;     // 32 KB per CTA and stage
constexpr int P_SMEM_BYTES = 1024 + P_STAGES * P_STAGE_BYTES + STAGING_BYTES + SMEM_AUX_BYTES;
constexpr int PBM = 256;                                         // rows per pair tile

template <int FMT, bool BIAS, bool PEERS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FFN_THREADS, 1)
ffn_grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                             const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmOut,
                             const __grid_constant__ PeerMapsArg<PEERS> peers, const FfnGemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t staging = ptx::smem_u32(smem + P_STAGES * P_STAGE_BYTES);
    uint8_t* aux = smem + P_STAGES * P_STAGE_BYTES + STAGING_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aux);             // full[S], empty[S], tfull[2], tempty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 132);
    int* prefix = reinterpret_cast<int*>(aux + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = ptx::cluster_ctarank();                   // 0 = the CTA that issues the MMAs
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const uint32_t bar_full = ptx::smem_u32(bars);                 // used in CTA 0 only
    const uint32_t bar_empty = bar_full + 8 * P_STAGES;            // one per CTA
    const uint32_t bar_tfull = bar_empty + 8 * P_STAGES;           // one per CTA
    const uint32_t bar_tempty = bar_tfull + 16;                    // used in CTA 0 only
    const uint32_t smem_base = ptx::smem_u32(smem);

    const int out_w = p.gated ? 128 : 256;
    const int n_tiles = (p.N + out_w - 1) / out_w;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, 8);                 // one elected lane of 4 epilogue warps x 2 CTAs
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        build_tile_prefix<PBM>(p, prefix, n_tiles, lane);
    } else if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::cluster_sync();               // both CTAs' barriers are initialised before anything signals them
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[p.groups];
    constexpr int bke = FMT == FMT_TF32 ? BK / 2 : BK;   // elements of K per stage: 128 bytes
    const int kblocks = p.K / bke;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB0);
            ptx::prefetch_tensormap(&tmB1);
            const CUtensorMap* tmB = (cta == 0) ? &tmB0 : &tmB1;
            const uint32_t full0 = ptx::mapa_shared(bar_full, 0);   // the full barriers live in CTA 0
            int stage = 0;
            uint32_t phase = 0;
            int vg = 0;
            uint32_t seen = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < total_tiles; tile += num_pairs) {
                const TileCoord t = decode_tile<PBM>(p, prefix, vg, tile, n_tiles, out_w);
                const int g = t.g, m0 = t.m0 + (int)cta * BM, n0 = t.n0;
                const int e = g % p.experts;
                const int nb = p.gated ? n0 : n0 + (int)cta * 128;
                ok = wait_source_rows(p, g, seen, abort_flag);
                if (!ok) break;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.dev_status);
                    if (!ok) break;
                    const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                    if (cta == 0) ptx::mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * P_STAGE_BYTES);
                    ptx::tma_load_3d_pair(sa, &tmA, kb * bke, m0, g, full0 + 8 * stage);
                    ptx::tma_load_3d_pair(sa + A_STAGE_BYTES, tmB, kb * bke, nb, e, full0 + 8 * stage);
                    if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (CTA 0 only)
        if (cta == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc_f32acc(PBM, BN, FMT == FMT_BF16 ? 1u : (FMT == FMT_F16 ? 0u : 2u));
            const uint32_t empty_peer = ptx::mapa_shared(bar_empty, 1);
            const uint32_t tfull_peer = ptx::mapa_shared(bar_tfull, 1);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < total_tiles; tile += num_pairs, ++it) {
                const int buf = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ok = ptx::mbar_wait_bounded(bar_tempty + 8 * buf, aphase ^ 1u, abort_flag, p.dev_status);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_full + 8 * stage, phase, abort_flag, p.dev_status);
                    if (!ok) break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                    const uint64_t da = ptx::umma_desc_k_sw128(sa);
                    const uint64_t db = ptx::umma_desc_k_sw128(sa + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        if constexpr (FMT == FMT_TF32) ptx::umma_tf32_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else ptx::umma_f16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    // release the stage in both CTAs
                    ptx::umma_commit_pair(bar_empty + 8 * stage);
                    ptx::umma_commit_pair(empty_peer + 8 * stage);
                    if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    ptx::umma_commit_pair(bar_tfull + 8 * buf);
                    ptx::umma_commit_pair(tfull_peer + 8 * buf);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const int epi_tid = threadIdx.x - 64;
        const uint32_t tempty0 = ptx::mapa_shared(bar_tempty, 0);
        int vg = 0;
        int it = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < total_tiles; tile += num_pairs, ++it) {
            const TileCoord t = decode_tile<PBM>(p, prefix, vg, tile, n_tiles, out_w);
            const int g = t.g, m0 = t.m0 + (int)cta * BM, n0 = t.n0;
            const int buf = it & 1;
            const uint32_t aphase = (it >> 1) & 1u;
            ok = ptx::mbar_wait_bounded(bar_tfull + 8 * buf, aphase, abort_flag, p.dev_status);
            ok = !ptx::named_barrier_or(2, EPI_THREADS, !ok);
            if (!ok) break;
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            const CUtensorMap* om = &tmOut;
            int og = g;
            uint8_t* md = nullptr;
            if constexpr (PEERS) {
                const int src = g / p.experts;
                om = &peers.m[src];
                og = p.peer_rank * p.experts + (g - src * p.experts);
                md = masked_peer_rows<FMT>(p, peers.base[src], og, g, m0, BM);
            }
            if constexpr (FMT == FMT_TF32)
                epilogue_tile_f32<true, BIAS, PEERS>(p, om, og, g, m0, n0, row_in_tile, taddr, tempty0 + 8 * buf, lane, epi_tid, staging, md);
            else
                epilogue_tile<true, FMT, BIAS, PEERS>(p, om, og, g, m0, n0, row_in_tile, taddr, tempty0 + 8 * buf, lane, epi_tid, staging, md);
        }
        if (epi_tid == 0) ptx::bulk_wait_group0();
    }

    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::cluster_sync();               // nobody leaves (or frees TMEM) while the other CTA may still signal it
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
// (outer, rows, K) tensor, K contiguous; box = 128 bytes x 128 rows x 1 with the 128-byte swizzle.
aristos_status_t make_map_3d(CUtensorMap* tm, const void* base, int K, int rows, int outer, int fmt) {
    const CUtensorMapDataType dt = fmt == FMT_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (fmt == FMT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    return encode_map_3d(tm, dt, fmt == FMT_TF32 ? 4 : 2, base, K, rows, outer, 128);
}

// Tile shapes. A single-CTA 128 x 256 tile stages 48 KB per 64-wide K block and is bound by the bandwidth that feeds
// the operands to the SM (tensor pipe 86-91 % active); a CTA pair (cta_group::2, 256 x 256 tile) stages 32 KB per SM
// for the same work (98-99 %). Pairs pad every group to whole 256-row tiles (128 wasted rows per group on average).
// The alternative - the pair kernel computes whole tiles only and a second, single-CTA launch finishes the < 256
// remaining rows of every group - wastes half as many rows but its few tiles fill their waves poorly: measured on
// 8 groups of about 4096 rows, the tail launches took 0.55 ms for 3 % of the rows and the two forms came out equal
// (8.04 against 8.08 ms of GEMM time per forward); the padded form needs half the launches.
//   TILES_AUTO    padded pairs where the row window holds at least 1024 rows, else single-CTA tiles
//   TILES_SINGLE  single-CTA tiles only
//   TILES_PAIR    pairs + single-CTA tail launch, for every window
//   TILES_PAIR_PADDED  padded pairs for every window
enum { TILES_AUTO = 0, TILES_SINGLE = 1, TILES_PAIR = 2, TILES_PAIR_PADDED = 3 };
int g_tile_mode = -1;      // -1: not yet read from the environment
int g_band_rows = -1;

int tile_mode() {
    if (g_tile_mode < 0) {
        const char* env = getenv("ARISTOS_FFN_TILES");
        g_tile_mode = !env ? TILES_AUTO
                           : (!strcmp(env, "single") ? TILES_SINGLE
                              : (!strcmp(env, "pair") ? TILES_PAIR
                                 : (!strcmp(env, "pair-padded") ? TILES_PAIR_PADDED : TILES_AUTO)));
    }
    return g_tile_mode;
}

// Rows per band of the tile order. A group whose A panel (rows x K) stays in L2 keeps the row-tile-fastest order
// (every B panel is then read from HBM once); a larger panel is walked in bands of 2048 rows, so that the CTAs of a
// wave share 2048 rows of A and about 8 B panels instead of re-reading the whole A panel for every few B panels.
// ARISTOS_FFN_BAND_ROWS overrides (0 = never band).
int band_rows_for(int window_rows, int K, int elt) {
    if (g_band_rows < 0) {
        const char* env = getenv("ARISTOS_FFN_BAND_ROWS");
        g_band_rows = env ? atoi(env) : 1;      // 1: automatic
        if (g_band_rows < 0) g_band_rows = 1;
    }
    if (g_band_rows != 1) return g_band_rows / 256 * 256;
    return (int64_t)window_rows * K * elt > (48ll << 20) ? 2048 : 0;
}

template <int FMT, bool BIAS, bool PEERS>
aristos_status_t max_pair_clusters(int* out) {
    // a persistent grid must be fully co-resident: ask how many 2-CTA clusters the device can hold at once
    static int max_clusters = -1;
    if (max_clusters < 0) {
        auto kernel = ffn_grouped_gemm_pair_kernel<FMT, BIAS, PEERS>;
        ARISTOS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES));
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(2 * (device_sm_count() / 2));
        lc.blockDim = dim3(FFN_THREADS);
        lc.dynamicSmemBytes = P_SMEM_BYTES;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
        lc.attrs = &at;
        lc.numAttrs = 1;
        int n = 0;
        ARISTOS_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &lc));
        max_clusters = n;
        if (getenv("ARISTOS_DEBUG")) fprintf(stderr, "[aristos] co-resident 2-CTA clusters: %d\n", n);
    }
    *out = max_clusters;
    return ARISTOS_OK;
}

template <int FMT, bool BIAS, bool PEERS>
aristos_status_t launch_gemm_t(const void* A, const void* B0, const void* B1, FfnGemmParams p, const PeerOutMaps& peers,
                               int grid_limit, cudaStream_t st) {
    CUtensorMap tmA, tmB0, tmB1, tmOut;
    ARISTOS_TRY(make_map_3d(&tmA, A, p.K, p.rows_per_group, p.groups, FMT));
    ARISTOS_TRY(make_map_3d(&tmB0, B0, p.K, p.N, p.experts, FMT));
    ARISTOS_TRY(make_map_3d(&tmB1, B1, p.K, p.N, p.experts, FMT));
    ARISTOS_TRY(make_map_3d(&tmOut, p.out, p.N, p.rows_per_group, p.groups, FMT));
    PeerMapsArg<PEERS> pm;
    if constexpr (PEERS) {
        memcpy(pm.m, peers.m, sizeof(pm.m));
        memcpy(pm.base, peers.base, sizeof(pm.base));
    } else {
        pm.unused = 0;
    }
    const int out_w = p.gated ? 128 : 256;
    int sms = device_sm_count();
    if (sms <= 0) { set_last_error("no CUDA device"); return ARISTOS_ERR_CUDA; }
    if (grid_limit > 0 && grid_limit < sms) sms = grid_limit;
    const int window = p.row_end - p.row_begin;
    const int band_rows = band_rows_for(window, p.K, FMT == FMT_TF32 ? 4 : 2);
    const int mode = tile_mode();
    const bool pairs = mode == TILES_PAIR || mode == TILES_PAIR_PADDED || (mode == TILES_AUTO && window >= 1024);
    const bool padded = mode != TILES_PAIR;
    if (pairs) {
        int max_clusters = 0;
        ARISTOS_TRY((max_pair_clusters<FMT, BIAS, PEERS>(&max_clusters)));
        const int64_t bound = (int64_t)p.groups * ceil_div(window, PBM) * ceil_div(p.N, out_w);
        int npairs = sms / 2 < max_clusters ? sms / 2 : max_clusters;
        if (bound < npairs) npairs = (int)bound;
        p.rows_mode = padded ? ROWS_ALL : ROWS_FULL_PAIRS;
        p.band = band_rows / PBM;
        if (npairs > 0 && (padded || window >= PBM)) {
            ffn_grouped_gemm_pair_kernel<FMT, BIAS, PEERS><<<2 * npairs, FFN_THREADS, P_SMEM_BYTES, st>>>(
                tmA, tmB0, tmB1, tmOut, pm, p);
            ARISTOS_COUNT_LAUNCH();
            ARISTOS_CUDA_TRY(cudaGetLastError());
        }
        if (padded) return ARISTOS_OK;
        p.rows_mode = ROWS_TAIL;     // the single-CTA kernel below finishes every group's last < 256 rows
    }
    auto kernel = ffn_grouped_gemm_kernel<FMT, BIAS, PEERS>;
    static bool attr_set = false;    // per instantiation
    if (!attr_set) {
        ARISTOS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set = true;
    }
    p.band = band_rows / BM;
    const int64_t bound = (int64_t)p.groups * (pairs ? 2 : ceil_div(window, BM)) * ceil_div(p.N, out_w);
    const int grid = (int)(bound < sms ? bound : sms);
    if (grid <= 0) return ARISTOS_OK;
    kernel<<<grid, FFN_THREADS, SMEM_BYTES, st>>>(tmA, tmB0, tmB1, tmOut, pm, p);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

// Both projections in one launch (ffn_updown_kernel). `done` holds groups * max_row_tiles counters.
template <int FMT, bool BIAS, bool PEERS>
aristos_status_t launch_updown_t(const void* xg, const void* w1, const void* w3, const void* h, const void* w2,
                                 const FfnGemmParams& p0, const FfnGemmParams& p1, const PeerOutMaps& peers,
                                 int32_t* done, int grid_limit, cudaStream_t st) {
    CUtensorMap tmA0, tmB00, tmB01, tmOut0, tmA1, tmB1, tmOut1;
    ARISTOS_TRY(make_map_3d(&tmA0, xg, p0.K, p0.rows_per_group, p0.groups, FMT));
    ARISTOS_TRY(make_map_3d(&tmB00, w1, p0.K, p0.N, p0.experts, FMT));
    ARISTOS_TRY(make_map_3d(&tmB01, w3, p0.K, p0.N, p0.experts, FMT));
    ARISTOS_TRY(make_map_3d(&tmOut0, p0.out, p0.N, p0.rows_per_group, p0.groups, FMT));
    ARISTOS_TRY(make_map_3d(&tmA1, h, p1.K, p1.rows_per_group, p1.groups, FMT));
    ARISTOS_TRY(make_map_3d(&tmB1, w2, p1.K, p1.N, p1.experts, FMT));
    ARISTOS_TRY(make_map_3d(&tmOut1, p1.out, p1.N, p1.rows_per_group, p1.groups, FMT));
    PeerMapsArg<PEERS> pm;
    if constexpr (PEERS) {
        memcpy(pm.m, peers.m, sizeof(pm.m));
        memcpy(pm.base, peers.base, sizeof(pm.base));
    } else {
        pm.unused = 0;
    }
    int sms = device_sm_count();
    if (sms <= 0) { set_last_error("no CUDA device"); return ARISTOS_ERR_CUDA; }
    if (grid_limit > 0 && grid_limit < sms) sms = grid_limit;
    const int window = p0.row_end - p0.row_begin;
    const int max_row_tiles = ceil_div(window, BM);
    auto kernel = ffn_updown_kernel<FMT, BIAS, PEERS>;
    static bool attr_set = false;
    if (!attr_set) {
        ARISTOS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set = true;
    }
    ARISTOS_CUDA_TRY(cudaMemsetAsync(done, 0, sizeof(int32_t) * (size_t)p0.groups * max_row_tiles, st));
    const int64_t bound = (int64_t)p0.groups * max_row_tiles * (ceil_div(p0.N, p0.gated ? 128 : 256) + ceil_div(p1.N, 256));
    const int grid = (int)(bound < sms ? bound : sms);
    if (grid <= 0) return ARISTOS_OK;
    kernel<<<grid, FFN_THREADS, SMEM_BYTES, st>>>(tmA0, tmB00, tmB01, tmOut0, tmA1, tmB1, tmOut1, pm, p0, p1, done,
                                                  max_row_tiles);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

template <int FMT>
aristos_status_t launch_updown_f(const void* xg, const void* w1, const void* w3, const void* h, const void* w2,
                                 const FfnGemmParams& p0, const FfnGemmParams& p1, const PeerOutMaps& peers,
                                 int32_t* done, int grid_limit, cudaStream_t st) {
    const bool bias = p0.bias0 || p0.bias1 || p1.bias0;
    const bool to_peers = p1.peer_world > 0;
    if (bias) return to_peers ? launch_updown_t<FMT, true, true>(xg, w1, w3, h, w2, p0, p1, peers, done, grid_limit, st)
                              : launch_updown_t<FMT, true, false>(xg, w1, w3, h, w2, p0, p1, peers, done, grid_limit, st);
    return to_peers ? launch_updown_t<FMT, false, true>(xg, w1, w3, h, w2, p0, p1, peers, done, grid_limit, st)
                    : launch_updown_t<FMT, false, false>(xg, w1, w3, h, w2, p0, p1, peers, done, grid_limit, st);
}

template <int FMT>
aristos_status_t launch_gemm_f(const void* A, const void* B0, const void* B1, const FfnGemmParams& p,
                               const PeerOutMaps& peers, int grid_limit, cudaStream_t st) {
    const bool bias = p.bias0 != nullptr || p.bias1 != nullptr;
    const bool to_peers = p.peer_world > 0;
    if (bias) return to_peers ? launch_gemm_t<FMT, true, true>(A, B0, B1, p, peers, grid_limit, st)
                              : launch_gemm_t<FMT, true, false>(A, B0, B1, p, peers, grid_limit, st);
    return to_peers ? launch_gemm_t<FMT, false, true>(A, B0, B1, p, peers, grid_limit, st)
                    : launch_gemm_t<FMT, false, false>(A, B0, B1, p, peers, grid_limit, st);
}

aristos_status_t launch_gemm(const void* A, const void* B0, const void* B1, const FfnGemmParams& p,
                             const PeerOutMaps& peers, int grid_limit, cudaStream_t st, int fmt) {
    switch (fmt) {
        case FMT_BF16: return launch_gemm_f<FMT_BF16>(A, B0, B1, p, peers, grid_limit, st);
        case FMT_F16: return launch_gemm_f<FMT_F16>(A, B0, B1, p, peers, grid_limit, st);
        default: return launch_gemm_f<FMT_TF32>(A, B0, B1, p, peers, grid_limit, st);
    }
}

}  // namespace

// Partly valid tiles of the fused return leave row by row, valid rows only (ARISTOS_EP_MASKED_RETURN=0: whole tiles
// by TMA store, padding rows included).
bool masked_return() {
    static int v = -1;
    if (v < 0) {
        const char* env = getenv("ARISTOS_EP_MASKED_RETURN");
        v = (env && !strcmp(env, "0")) ? 0 : 1;
    }
    return v == 1;
}

void ffn_set_tile_mode(int mode) { g_tile_mode = (mode >= TILES_AUTO && mode <= TILES_PAIR_PADDED) ? mode : -1; }
int ffn_tile_mode() { return tile_mode(); }

aristos_status_t expert_ffn_tc_sm100(const void* xg, const int32_t* count, int groups, int rows_per_group,
                                        int experts, const void* w1, const void* w3, const void* w2, const void* b1,
                                        const void* b3, const void* b2, void* h_scratch, void* y, int H, int I,
                                        int hidden_act, int fmt, int row_begin, int row_end, int sm_limit,
                                        int32_t* dev_status, cudaStream_t st, const FfnEpArgs* ep) {
    const int peer_world = ep ? ep->peer_world : 0;
    if (peer_world > MAX_PEER_OUT || (peer_world > 0 && (!ep->peer_y || groups != peer_world * experts))) {
        set_last_error("expert_ffn: peer output needs world <= %d and groups == world * experts", MAX_PEER_OUT);
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (ep && ep->src_flags && (experts <= 0 || groups / experts > 32)) {
        set_last_error("expert_ffn: arrival flags need at most 32 source ranks");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (groups > MAX_GROUPS) { set_last_error("expert_ffn: more than %d row groups", MAX_GROUPS); return ARISTOS_ERR_CONFIG; }
    if (H % BK != 0 || I % BK != 0) { set_last_error("expert_ffn: H and I must be multiples of 64"); return ARISTOS_ERR_CONFIG; }
    if (row_begin % BM != 0) { set_last_error("expert_ffn: row_begin must be a multiple of 128"); return ARISTOS_ERR_INVALID_ARG; }
    const bool gated = hidden_act == ARISTOS_ACT_SWIGLU;
    FfnGemmParams p{};
    p.count = count;
    p.groups = groups;
    p.experts = experts;
    p.rows_per_group = rows_per_group;
    p.row_begin = row_begin;
    p.row_end = row_end;
    p.dev_status = dev_status;
    p.self_source = -1;
    if (ep) {
        p.first_source = ep->first_source;
        p.src_flags = ep->src_flags;
        p.flag_epoch = ep->flag_epoch;
        p.flag_limit_ms = ep->flag_limit_ms > 0 ? ep->flag_limit_ms : 2000;
        p.self_source = ep->self_source;
    }
    // up-projection: h = epi(xg * W1^T [, xg * W3^T])
    p.N = I;
    p.K = H;
    p.gated = gated ? 1 : 0;
    p.act = hidden_act;
    p.out = h_scratch;
    p.bias0 = b1;
    p.bias1 = gated ? b3 : nullptr;
    static const PeerOutMaps no_peers{};
    // small row groups: both projections in one persistent launch (needs the caller's counter scratch)
    const int window = row_end - row_begin;
    const int mode = tile_mode();
    const bool small_groups = mode == TILES_SINGLE || (mode == TILES_AUTO && window < 1024);
    const char* fz = getenv("ARISTOS_FFN_FUSED");
    const bool one_launch = small_groups && ep && ep->updown_scratch &&
                            ep->updown_scratch_ints >= (size_t)groups * ceil_div(window, BM) && !(fz && !strcmp(fz, "0")) &&
                            !(mode == TILES_SINGLE && !(fz && !strcmp(fz, "1")));
    const FfnGemmParams p_up = p;
    if (!one_launch) ARISTOS_TRY(launch_gemm(xg, w1, gated ? w3 : w1, p, no_peers, sm_limit, st, fmt));
    // down-projection: y = h * W2^T (h was written by the launch above: nothing left to wait for)
    p.src_flags = nullptr;
    p.N = H;
    p.K = I;
    p.gated = 0;
    p.act = ARISTOS_ACT_IDENTITY;
    p.out = y;
    p.bias0 = b2;
    p.bias1 = nullptr;
    if (one_launch) {
        PeerOutMaps peers{};
        if (peer_world > 0) {
            for (int d = 0; d < peer_world; ++d) {
                ARISTOS_TRY(make_map_3d(&peers.m[d], ep->peer_y[d], H, rows_per_group, peer_world * experts, fmt));
                peers.base[d] = masked_return() ? ep->peer_y[d] : nullptr;
            }
            p.peer_world = peer_world;
            p.peer_rank = ep->peer_rank;
        }
        const void* w3x = gated ? w3 : w1;
        switch (fmt) {
            case FMT_BF16: return launch_updown_f<FMT_BF16>(xg, w1, w3x, h_scratch, w2, p_up, p, peers, ep->updown_scratch, sm_limit, st);
            case FMT_F16: return launch_updown_f<FMT_F16>(xg, w1, w3x, h_scratch, w2, p_up, p, peers, ep->updown_scratch, sm_limit, st);
            default: return launch_updown_f<FMT_TF32>(xg, w1, w3x, h_scratch, w2, p_up, p, peers, ep->updown_scratch, sm_limit, st);
        }
    }
    if (peer_world > 0) {
        // every source rank's return buffer holds (all experts, rows_per_group, H); rows of group (src, e_local) land
        // in rank src's block peer_rank * experts + e_local
        PeerOutMaps peers{};
        for (int d = 0; d < peer_world; ++d) {
            ARISTOS_TRY(make_map_3d(&peers.m[d], ep->peer_y[d], H, rows_per_group, peer_world * experts, fmt));
            peers.base[d] = masked_return() ? ep->peer_y[d] : nullptr;
        }
        p.peer_world = peer_world;
        p.peer_rank = ep->peer_rank;
        ARISTOS_TRY(launch_gemm(h_scratch, w2, w2, p, peers, sm_limit, st, fmt));
        return ARISTOS_OK;
    }
    ARISTOS_TRY(launch_gemm(h_scratch, w2, w2, p, no_peers, sm_limit, st, fmt));
    return ARISTOS_OK;
}

}  // namespace aristos
