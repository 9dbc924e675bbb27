// Expert FFN with FP8 (e4m3) operands and fp32 block scales on the 5th-generation tensor cores.
//
// Operands: activations quantised per row and per 128 elements of K (scale sa[row][K/128]), weights quantised per
// 128 x 128 block (scale sb[expert][N/128][K/128]); out = sum over K blocks kb of sa[row,kb] * sb[n/128,kb] *
// (Aq[row, kb] . Bq[n, kb]). The hardware's own block scaling (power-of-two scales per 32 elements) cannot express
// fp32 scales per 128, so the accumulation has two levels: one 128-wide K block is accumulated by four
// tcgen05.mma kind::f8f6f4 (M128 x N256 x K32 each) into a fresh 256-column TMEM accumulator, eight promotion warps
// drain it (tcgen05.ld, 16 columns at a time, one load in flight while the previous one is used), multiply by the
// block's scale and add it to fp32 register accumulators with packed FMAs while the tensor core fills the other of
// the two TMEM buffers. Two promotion warps share a TMEM lane quarter, each owning four of the eight 32-column chunks
// ({0, 2, 4, 6} or {1, 3, 5, 7}, so a SwiGLU thread holds matching gate and up columns): one row and 128 columns per
// thread. Two issuing warps take turns per K block (a commit covers its own thread's MMAs only).
//
// What bounds the kernel: every K block's 128 x 256 fp32 partial sums (128 KB) have to leave TMEM through tcgen05.ld.
// Clock stamps inside the kernel (per K block, CTA 0) showed a promotion warp needing about 1050 cycles for its share
// of a block (~260 per 32 columns with the two warps of a lane quarter loading at once, i.e. roughly 32 bytes per
// clock and lane quarter, 128 per SM), the same whether the tensor core was running beside it or idle, with 16- or
// 32-column loads, one or two loads in flight, and with the registers of the other warps handed to the promotion
// warps; issuing a block's MMAs cost 85 cycles and the operands were never late (75 cycles waiting for TMA). The
// tensor core needs 542 cycles for the block, so it can be busy about half of the time (measured: 51 % in the up
// projection): the format's fp32 scale per 128 elements of K, not the MMA rate, sets the speed of this kernel.
// (A variant with four promotion warps per lane quarter that took their registers from the other warps with
// setmaxnreg did not finish on the GPU and was not run again; with two per quarter the hand-over changed nothing.)
//
// Same tile contract as the 16-bit kernel (ffn_sm100.cu; reference: fGET, mma.cuh:46-179, A (M,K) and B (N,K)
// row-major, epilogue act(acc)): persistent CTAs, warp 0 = TMA producer (a 128-byte K block is exactly one swizzled
// row; four 48 KB stages), warps 1 and 10 = MMA issuers, warps 2-9 = promotion + epilogue. SwiGLU tiles hold 128 gate
// and 128 up columns in one N = 256 instruction. The down projection's output is bf16, written with 16-byte stores
// masked by the group's row count (to this rank's buffer, or straight into the source ranks' buffers through peer
// pointers). The up projection's output feeds the down projection as e4m3: its epilogue rounds to bf16, takes each
// row's amax over the 128-column scale group (held half and half by the two promotion warps of a lane quarter, which
// meet on an mbarrier with a bounded wait) and writes codes and scales of the valid rows - the same bits as
// quantising a bf16 copy afterwards, without the copy.
#include <cuda.h>
#include <cuda_fp8.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tensor_map.cuh"

namespace aristos {

namespace {

constexpr int F8_BM = 128;
constexpr int F8_BN = 256;                       // MMA N = TMEM columns per accumulator buffer
constexpr int F8_KB = 128;                       // elements (= bytes) of K per stage and per scale block
constexpr int F8_STAGES = 4;
constexpr int F8_A_BYTES = F8_BM * F8_KB;        // 16 KB
constexpr int F8_B_BYTES = F8_BN * F8_KB;        // 32 KB: two boxes of 128 weight rows
constexpr int F8_STAGE_BYTES = F8_A_BYTES + F8_B_BYTES;
constexpr int F8_TBUFS = 2;                      // TMEM accumulator buffers (2 x 256 columns)
// Promotion warps per TMEM lane quarter: each owns 8 / SUBS of the eight 32-column chunks of the 256-column tile
// (chunks sub, sub + SUBS, ...). Roles: warp 0 producer, warp 1 MMA, warps 2 .. 2 + 4 SUBS promotion, then the second MMA
// warp. Two per quarter is the measured optimum: with four, 608 threads leave 96 registers each and the kernel slows down.
constexpr int f8_threads(int subs) { return 32 * (3 + 4 * subs); }
constexpr int F8_MAX_GROUPS = 1024;
constexpr int F8_AUX_BYTES = 256 + (F8_MAX_GROUPS + 1) * 4;
constexpr int F8_AUX_ALIGNED = (F8_AUX_BYTES + 127) & ~127;
constexpr int F8_QSTAGE_BYTES_PER_WARP = 2048;               // output staging per promotion warp: 16 rows x 128 bytes of
                                                             // bf16 (plain output) or 32 rows x 32 codes (quantised)
constexpr int F8_AMAX_BYTES = 2 * 2 * 128 * 2 * 4;           // [tile parity][scale group][row][warp of the pair]
constexpr int F8_SMEM_BYTES = 1024 + F8_STAGES * F8_STAGE_BYTES + F8_AUX_ALIGNED + 8 * F8_QSTAGE_BYTES_PER_WARP +
                              F8_AMAX_BYTES;
static_assert(F8_SMEM_BYTES <= 227 * 1024, "fp8 GEMM: shared memory");

struct Fp8GemmParams {
    const int32_t* count;
    int groups, experts, rows_per_group, row_begin, row_end;
    int N, K;
    int gated, act;
    const float* sa;      // [groups * rows_per_group][K / 128]
    const float* sb0;     // [experts][ceil(N / 128)][K / 128]
    const float* sb1;     // SwiGLU: scales of the up projection's weights
    __nv_bfloat16* out;   // [groups * rows_per_group][N]
    int32_t* dev_status;
    // quantised output (up projection): e4m3 codes [groups * rows_per_group][N] and one fp32 scale per row and 128
    // columns, bit for bit what quantising the bf16 output afterwards would give; `out` is not written then
    uint8_t* outq;
    float* out_scales;
};
static_assert(sizeof(Fp8GemmParams) <= 128, "Fp8GemmParams: keep the kernel argument within 128 bytes");

// Expert-parallel output, a kernel argument of its own (the hot parameters above stay within 128 bytes: a larger
// struct changes how the compiler treats the argument).
struct Fp8PeerArgs {
    // peer_world > 0: rows of group g = src * experts + e are stored into rank src's buffer peer_out[src]
    // ((peer_world * experts, rows_per_group, N), mapped into this process) as group peer_rank * experts + e
    int peer_world, peer_rank;
    __nv_bfloat16* peer_out[8];
    // Dense groups (src_off != nullptr; groups == experts): group e holds the rows of every source rank back to back,
    // source s in rows [src_off[e * (peer_world + 1) + s], src_off[... + s + 1]); row r of source s returns to rank s
    // as row r - src_off[..s] of its group peer_rank * experts + e, whose groups have ret_rows rows.
    const int32_t* src_off;
    int ret_rows;
};

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// e4m3 x e4m3 -> fp32, both operands K-major, tile M x N (formats 0 = e4m3 in bits 7-9 and 10-12).
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int M, int N) {
    return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
}

// Where output row `row` of group g goes (column 0 of the N-wide row): this rank's buffer, or - expert parallel - the
// buffer of the rank the row came from, in that rank's own numbering.
__device__ __forceinline__ __nv_bfloat16* fp8_output_row(const Fp8GemmParams& p, const Fp8PeerArgs& pa, int g, int row) {
    __nv_bfloat16* obase = p.out;
    int og = g;
    int orows = p.rows_per_group, orow_idx = row;
    if (pa.peer_world > 0 && pa.src_off != nullptr) {
        // dense group: find the source rank of this row, return it to that rank's own numbering
        const int32_t* off = pa.src_off + g * (pa.peer_world + 1);
        int src = 0;
        while (src + 1 < pa.peer_world && row >= __ldg(off + src + 1)) ++src;
        obase = pa.peer_out[src];
        og = pa.peer_rank * p.experts + g;
        orows = pa.ret_rows;
        orow_idx = row - __ldg(off + src);
    } else if (pa.peer_world > 0) {        // the store is the return all-to-all: straight into the source rank
        const int src = g / p.experts;
        obase = pa.peer_out[src];
        og = pa.peer_rank * p.experts + (g - src * p.experts);
    }
    return obase + ((size_t)og * orows + orow_idx) * p.N;
}

template <int SUBS, bool QUANT>
__global__ void __launch_bounds__(f8_threads(SUBS), 1)
ffn_fp8_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                            const __grid_constant__ CUtensorMap tmB1, const Fp8GemmParams p,
                            const __grid_constant__ Fp8PeerArgs pa) {
    constexpr int F8_EPI_THREADS = 128 * SUBS;
    constexpr int CH = 8 / SUBS;                           // 32-column chunks per promotion thread
    constexpr int MMA2_WARP = 2 + 4 * SUBS;
    static_assert(!QUANT || SUBS == 2, "the quantising epilogue pairs the two promotion warps of a lane quarter");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* aux = smem + F8_STAGES * F8_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aux);     // full[S], empty[S], tfull[2], tempty[2], amax[4]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 196);
    int* prefix = reinterpret_cast<int*>(aux + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * F8_STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * F8_STAGES;
    const uint32_t bar_tempty = bar_tfull + 8 * F8_TBUFS;
    const uint32_t bar_amax = bar_tempty + 8 * F8_TBUFS;   // where the two promotion warps of a lane quarter meet
    const uint32_t smem_base = ptx::smem_u32(smem);

    const int out_w = p.gated ? 128 : 256;
    const int n_tiles = (p.N + out_w - 1) / out_w;
    const int window = p.row_end - p.row_begin;
    const int kblocks = p.K / F8_KB;
    const int nblk = (p.N + 127) / 128;                    // weight-scale blocks along N

    if (threadIdx.x == 0) {
        for (int s = 0; s < F8_STAGES; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < F8_TBUFS; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, F8_EPI_THREADS);
        }
        for (int q = 0; q < 4; ++q) ptx::mbar_init(bar_amax + 8 * q, 64);
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        int running = 0;
        if (lane == 0) prefix[0] = 0;
        for (int g0 = 0; g0 < p.groups; g0 += 32) {
            const int g = g0 + lane;
            int v = 0;
            if (g < p.groups) {
                int rows = p.count[ordered_group(g, p.groups, p.experts)] - p.row_begin;
                rows = max(0, min(rows, window));
                v = ((rows + F8_BM - 1) / F8_BM) * n_tiles;
            }
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, v, d);
                if (lane >= d) v += o;
            }
            if (g < p.groups) prefix[g + 1] = running + v;
            running += __shfl_sync(0xffffffffu, v, 31);
        }
    } else if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), F8_TBUFS * F8_BN);
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[p.groups];

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB0);
            ptx::prefetch_tensormap(&tmB1);
            int stage = 0;
            uint32_t phase = 0;
            int vg = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                while (tile >= prefix[vg + 1]) ++vg;
                const int g = ordered_group(vg, p.groups, p.experts);
                const int local = tile - prefix[vg];
                const int mt = (prefix[vg + 1] - prefix[vg]) / n_tiles;
                const int m0 = p.row_begin + (local % mt) * F8_BM;
                const int n0 = (local / mt) * out_w;
                const int e = g % p.experts;
                const int n1 = p.gated ? n0 : n0 + 128;     // second 128-row box of B
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.dev_status);
                    if (!ok) break;
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * F8_STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(full, F8_STAGE_BYTES);
                    ptx::tma_load_3d(sa, &tmA, kb * F8_KB, m0, g, full);
                    ptx::tma_load_3d(sa + F8_A_BYTES, &tmB0, kb * F8_KB, n0, e, full);
                    ptx::tma_load_3d(sa + F8_A_BYTES + F8_B_BYTES / 2, &tmB1, kb * F8_KB, n1, e, full);
                    if (++stage == F8_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == MMA2_WARP) {
        // ------------------------------------------------------------------ MMA issuers: one TMEM buffer per K block.
        // Issuing the four MMAs and the commit of one K block costs the issuing thread more cycles than the tensor
        // core needs to run them, so two warps take turns: K block number it goes to warp it % 2 and to TMEM buffer
        // it % 2 (each thread's commit covers its own MMAs only).
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = umma_idesc_e4m3(F8_BM, F8_BN);
            const int me = warp == 1 ? 0 : 1;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    if ((it & 1) != me) continue;
                    const int tbuf = it & 1, stage = it % F8_STAGES;
                    const uint32_t tphase = (it >> 1) & 1u, phase = (it / F8_STAGES) & 1u;
                    ok = ptx::mbar_wait_bounded(bar_tempty + 8 * tbuf, tphase ^ 1u, abort_flag, p.dev_status);
                    if (!ok) break;
                    ok = ptx::mbar_wait_bounded(bar_full + 8 * stage, phase, abort_flag, p.dev_status);
                    if (!ok) break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * F8_STAGE_BYTES;
                    const uint64_t da = ptx::umma_desc_k_sw128(sa);
                    const uint64_t db = ptx::umma_desc_k_sw128(sa + F8_A_BYTES);
                    const uint32_t tmem_d = tmem_base + tbuf * F8_BN;
#pragma unroll
                    for (int k = 0; k < 4; ++k)            // K = 32 elements = 32 bytes per instruction
                        umma_f8(tmem_d, da + 2 * k, db + 2 * k, idesc, k != 0 ? 1u : 0u);
                    // one commit: the accumulator is ready; the promotion warps hand the stage back when they see it
                    ptx::umma_commit(bar_tfull + 8 * tbuf);
                }
            }
        }
        __syncwarp();
    } else if (warp >= 2 && warp < MMA2_WARP) {
        // ------------------------------------------------------------------ promotion + epilogue
        // A thread owns one accumulator row and the CH 32-column chunks half, half + SUBS, ... of the 256-column tile:
        // the first CH / 2 lie in the tile's first 128 columns (gate, or weight-scale block n0 / 128), the others in
        // the second 128 (up, or the next scale block).
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;                   // 0 .. SUBS - 1
        const int row_in_tile = quarter * 32 + lane;
        int vg = 0, tbuf = 0, rstage = 0;
        int qtile = 0;                                      // tiles quantised so far (parity of the amax buffer)
        uint32_t tphase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
            while (tile >= prefix[vg + 1]) ++vg;
            const int g = ordered_group(vg, p.groups, p.experts);
            const int local = tile - prefix[vg];
            const int mt = (prefix[vg + 1] - prefix[vg]) / n_tiles;
            const int m0 = p.row_begin + (local % mt) * F8_BM;
            const int n0 = (local / mt) * out_w;
            const int e = g % p.experts;
            const int row = m0 + row_in_tile;
            const int row_limit = min(p.count[g], p.row_end);
            const bool row_ok = row < row_limit;
            const float* sa_row = p.sa + ((size_t)g * p.rows_per_group + min(row, p.rows_per_group - 1)) * kblocks;
            const int blk = n0 / 128;
            const float* sb0_row = p.sb0 + ((size_t)e * nblk + blk) * kblocks;
            const float* sb1_row = p.gated ? p.sb1 + ((size_t)e * nblk + blk) * kblocks
                                           : p.sb0 + ((size_t)e * nblk + min(blk + 1, nblk - 1)) * kblocks;
            // Which 32-column chunks a thread owns: SwiGLU tiles and the quantising epilogue interleave the warps of a
            // lane quarter (chunk j of a thread = half + SUBS j), so a thread holds matching gate / up columns or half
            // of each scale group; plain output gives every thread CH adjacent chunks (256 / SUBS contiguous columns),
            // so that its row leaves in whole 128-byte lines. The sums per output element are the same either way.
            const bool contig = !QUANT && !p.gated;
            const uint32_t cbase = contig ? half * (256 / SUBS) : half * 32;
            const uint32_t cstride = contig ? 32 : 32 * SUBS;
            float2 acc[CH][16];                              // chunk j at columns cbase + j * cstride, as 16 pairs
#pragma unroll
            for (int j = 0; j < CH; ++j)
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[j][i] = make_float2(0.0f, 0.0f);
            for (int kb = 0; kb < kblocks; ++kb) {
                const float sa = __ldg(sa_row + kb);
                const float w_lo = sa * __ldg(sb0_row + kb);       // columns 0..127
                const float w_hi = sa * __ldg(sb1_row + kb);       // columns 128..255
                ok = ptx::mbar_wait_bounded(bar_tfull + 8 * tbuf, tphase, abort_flag, p.dev_status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // the MMAs of this K block are complete, so their shared-memory stage is free again
                if (threadIdx.x == 64) ptx::mbar_arrive(bar_empty + 8 * rstage);
                if (++rstage == F8_STAGES) rstage = 0;
                ptx::tcgen05_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + tbuf * F8_BN + cbase;
                // 2 CH 16-column loads, one in flight while the previous one is accumulated
                uint32_t v[2][16];
                ptx::tmem_ld_32x32b_x16(taddr, v[0]);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int s = 0; s < 2 * CH; ++s) {
                    if (s + 1 < 2 * CH)
                        ptx::tmem_ld_32x32b_x16(taddr + ((s + 1) >> 1) * cstride + ((s + 1) & 1) * 16, v[(s + 1) & 1]);
                    const float w = cbase + (s >> 1) * cstride < 128 ? w_lo : w_hi;
                    const float2 w2 = make_float2(w, w);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float2 x2 = make_float2(__uint_as_float(v[s & 1][2 * i]), __uint_as_float(v[s & 1][2 * i + 1]));
                        acc[s >> 1][(s & 1) * 8 + i] = __ffma2_rn(x2, w2, acc[s >> 1][(s & 1) * 8 + i]);
                    }
                    if (s + 1 < 2 * CH) {
                        ptx::tmem_ld_wait();
                    } else {
                        ptx::tcgen05_fence_before();
                        ptx::mbar_arrive(bar_tempty + 8 * tbuf);   // drained: the tensor core may refill the buffer
                    }
                }
                if (++tbuf == F8_TBUFS) { tbuf = 0; tphase ^= 1u; }
            }
            if (!ok) break;
            if constexpr (QUANT) {
                // ---- epilogue, quantised: the tile's 128 (SwiGLU) or 2 x 128 output columns of a row are one or two
                // scale groups, split between the two warps of the lane quarter: amax through shared memory
                float amax[2] = {0.0f, 0.0f};              // the activated bf16 values replace acc[j] in place
                const int nchunks = p.gated ? 2 : 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j >= nchunks) break;
                    const int ju = (j + 2) & 3;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float v0, v1;
                        if (p.gated) {
                            v0 = act_silu(acc[j][i].x) * acc[ju][i].x;
                            v1 = act_silu(acc[j][i].y) * acc[ju][i].y;
                        } else {
                            v0 = acc[j][i].x;
                            v1 = acc[j][i].y;
                            if (p.act == ARISTOS_ACT_RELU) { v0 = act_relu(v0); v1 = act_relu(v1); }
                            else if (p.act == ARISTOS_ACT_GELU) { v0 = act_gelu(v0); v1 = act_gelu(v1); }
                        }
                        const __nv_bfloat162 r = __floats2bfloat162_rn(v0, v1);     // the bf16 value is what is quantised
                        acc[j][i] = make_float2(__low2float(r), __high2float(r));
                        const int b = p.gated ? 0 : (j >> 1);
                        amax[b] = fmaxf(amax[b], fmaxf(fabsf(acc[j][i].x), fabsf(acc[j][i].y)));
                    }
                }
                float* ex = reinterpret_cast<float*>(aux + F8_AUX_ALIGNED + 8 * F8_QSTAGE_BYTES_PER_WARP) + (qtile & 1) * 512;
                const uint32_t out_stage = ptx::smem_u32(aux + F8_AUX_ALIGNED) + (warp - 2) * F8_QSTAGE_BYTES_PER_WARP;
                ex[row_in_tile * 2 + half] = amax[0];
                ex[256 + row_in_tile * 2 + half] = amax[1];
                ptx::mbar_arrive(bar_amax + 8 * quarter);
                ok = ptx::mbar_wait_bounded(bar_amax + 8 * quarter, qtile & 1, abort_flag, p.dev_status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                amax[0] = fmaxf(amax[0], ex[row_in_tile * 2 + (half ^ 1)]);
                amax[1] = fmaxf(amax[1], ex[256 + row_in_tile * 2 + (half ^ 1)]);
                ++qtile;
                const size_t grow = (size_t)g * p.rows_per_group + row;
                uint8_t* my_q = row_ok ? p.outq + grow * p.N + n0 : nullptr;
                uint8_t* q2[2];                              // rows it * 16 + lane / 2 of this warp's 32
#pragma unroll
                for (int it = 0; it < 2; ++it)
                    q2[it] = reinterpret_cast<uint8_t*>(
                        __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_q), it * 16 + (lane >> 1)));
                const int unit = lane & 1;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    if (b == 1 && p.gated) break;
                    if (n0 + b * 128 >= p.N) break;
                    const float scale = amax[b] > 0.0f ? amax[b] / 448.0f : 1.0f;
                    const float inv = 1.0f / scale;
                    if (row_ok && half == 0) p.out_scales[grow * nblk + blk + b] = scale;
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int j = p.gated ? jj : 2 * b + jj;
                        if (j >= 4) break;
                        const int col = (half + 2 * j) * 32;
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            o[i] = 0;
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const float2 pr = acc[j][2 * i + (c >> 1)];
                                o[i] |= (uint32_t)__nv_cvt_float_to_fp8(((c & 1) ? pr.y : pr.x) * inv, __NV_SATFINITE, __NV_E4M3) << (8 * c);
                            }
                        }
                        // row `lane`, 16-byte unit u lands at unit u ^ ((lane / 4) % 2): no bank conflicts either way
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            ptx::st_shared_v4(out_stage + lane * 32 + ((u ^ ((lane >> 2) & 1)) << 4), o[4 * u], o[4 * u + 1],
                                              o[4 * u + 2], o[4 * u + 3]);
                        __syncwarp();
#pragma unroll
                        for (int it = 0; it < 2; ++it) {
                            const int r = it * 16 + (lane >> 1);
                            const uint4 val = ptx::ld_shared_v4(out_stage + r * 32 + ((unit ^ ((r >> 2) & 1)) << 4));
                            if (q2[it] != nullptr) *reinterpret_cast<uint4*>(q2[it] + col + unit * 16) = val;
                        }
                        __syncwarp();
                    }
                }
            } else {
            if (row_ok && (p.gated || SUBS != 2)) {
                __nv_bfloat16* orow = fp8_output_row(p, pa, g, row) + n0;
                if (p.gated) {
                    // gate chunk half + SUBS j pairs with up chunk half + SUBS j + 4: 32 outputs each
#pragma unroll
                    for (int j = 0; j < CH / 2; ++j) {
                        const int col = (half + SUBS * j) * 32;
                        if (n0 + col >= p.N) break;
                        uint32_t o[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            o[i] = pack_bf16x2(act_silu(acc[j][i].x) * acc[j + CH / 2][i].x,
                                               act_silu(acc[j][i].y) * acc[j + CH / 2][i].y);
                        uint4* dst = reinterpret_cast<uint4*>(orow + col);
#pragma unroll
                        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                    }
                } else if (SUBS != 2) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int col = cbase + j * 32;
                        if (n0 + col >= p.N) break;
                        uint32_t o[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float v0 = acc[j][i].x, v1 = acc[j][i].y;
                            if (p.act == ARISTOS_ACT_RELU) { v0 = act_relu(v0); v1 = act_relu(v1); }
                            else if (p.act == ARISTOS_ACT_GELU) { v0 = act_gelu(v0); v1 = act_gelu(v1); }
                            o[i] = pack_bf16x2(v0, v1);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(orow + col);
#pragma unroll
                        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                    }
                }
            }
            if (!QUANT && !p.gated && SUBS == 2 && n0 + (int)cbase < p.N) {
                // Plain output, two promotion warps per lane quarter: a thread holds 128 adjacent columns (256 bytes)
                // of its row. The rows leave through the warp's staging area, 16 rows x 128 bytes at a time, so that a
                // store instruction writes four whole 128-byte lines (local memory, or a peer's over NVLink) instead
                // of 32 separate 16-byte pieces.
                __nv_bfloat16* my_dst = nullptr;             // where this lane's row goes (column n0 + cbase), if valid
                if (row_ok) my_dst = fp8_output_row(p, pa, g, row) + n0 + cbase;
                const uint32_t out_stage = ptx::smem_u32(aux + F8_AUX_ALIGNED) + (warp - 2) * F8_QSTAGE_BYTES_PER_WARP;
                const int unit = lane & 7;
#pragma unroll
                for (int jp = 0; jp < CH / 2; ++jp) {        // chunks 2 jp and 2 jp + 1: 64 columns = one 128-byte line
                    uint32_t o[32];
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float v0 = acc[2 * jp + jj][i].x, v1 = acc[2 * jp + jj][i].y;
                            if (p.act == ARISTOS_ACT_RELU) { v0 = act_relu(v0); v1 = act_relu(v1); }
                            else if (p.act == ARISTOS_ACT_GELU) { v0 = act_gelu(v0); v1 = act_gelu(v1); }
                            o[jj * 16 + i] = pack_bf16x2(v0, v1);
                        }
#pragma unroll
                    for (int hr = 0; hr < 2; ++hr) {         // lanes 0-15, then lanes 16-31
                        if ((lane >> 4) == hr) {
                            const int r = lane & 15;
#pragma unroll
                            for (int u = 0; u < 8; ++u)      // 16-byte unit u of row r lands at unit u ^ (r % 8)
                                ptx::st_shared_v4(out_stage + r * 128 + ((u ^ (r & 7)) << 4), o[4 * u], o[4 * u + 1],
                                                  o[4 * u + 2], o[4 * u + 3]);
                        }
                        __syncwarp();
#pragma unroll
                        for (int it = 0; it < 4; ++it) {
                            const int r = it * 4 + (lane >> 3);  // staged row; lane hr * 16 + r of the warp owns it
                            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(
                                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_dst), hr * 16 + r));
                            const uint4 val = ptx::ld_shared_v4(out_stage + r * 128 + ((unit ^ (r & 7)) << 4));
                            if (dst != nullptr) *reinterpret_cast<uint4*>(dst + jp * 64 + unit * 8) = val;
                        }
                        __syncwarp();
                    }
                }
            }
            }
        }
    }

    ptx::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, F8_TBUFS * F8_BN);
    }
}

// ---- quantisation ------------------------------------------------------------------------------------------------
// Quantise 128 consecutive elements held 4 per lane by one warp: scale = amax / 448 (1 when all zero).
template <typename T>
__device__ __forceinline__ void quantize_group128(const T* __restrict__ s, uint8_t* __restrict__ d,
                                                  float* __restrict__ scale_out, int lane) {
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = static_cast<float>(s[lane * 4 + i]);
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        packed |= (uint32_t)__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * i);
    *reinterpret_cast<uint32_t*>(d + lane * 4) = packed;
    if (lane == 0) *scale_out = scale;
}

// Every row of a (rows, cols) tensor: one warp per (row, 128-column group).
template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_fp8_kernel(const T* __restrict__ src, int64_t rows, int cols, uint8_t* __restrict__ dst,
                         float* __restrict__ scales) {
    const int ngroup = cols / 128;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t task = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; task < rows * ngroup; task += nwarps) {
        const int64_t row = task / ngroup;
        const int cg = (int)(task % ngroup);
        quantize_group128(src + row * cols + cg * 128, dst + row * cols + cg * 128, scales + row * ngroup + cg, lane);
    }
}

// Only the valid rows of a (groups, rows_per_group, cols) tensor (row < count[group]): a persistent grid walks the
// flattened list of valid (row, column group) pairs, found through a prefix over the groups' counts.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_group_rows_fp8_kernel(const T* __restrict__ src, const int32_t* __restrict__ count, int groups,
                               int rows_per_group, int cols, uint8_t* __restrict__ dst, float* __restrict__ scales) {
    __shared__ int s_prefix[F8_MAX_GROUPS + 1];
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int running = 0;
        if (lane == 0) s_prefix[0] = 0;
        for (int g0 = 0; g0 < groups; g0 += 32) {
            const int g = g0 + lane;
            int v = g < groups ? min(max(count[g], 0), rows_per_group) : 0;
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
    const int ngroup = cols / 128;
    const int lane = threadIdx.x & 31;
    const int64_t total = (int64_t)s_prefix[groups] * ngroup;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t task = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; task < total; task += nwarps) {
        const int vrow = (int)(task / ngroup);
        const int cg = (int)(task % ngroup);
        int lo = 0, hi = groups;                       // largest g with s_prefix[g] <= vrow
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_prefix[mid] <= vrow) lo = mid; else hi = mid;
        }
        const int64_t row = (int64_t)lo * rows_per_group + (vrow - s_prefix[lo]);
        quantize_group128(src + row * cols + cg * 128, dst + row * cols + cg * 128, scales + row * ngroup + cg, lane);
    }
}

// One CTA per 128 x 128 block of a (mats, rows, cols) tensor: scale = amax / 448.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_blocks_fp8_kernel(const T* __restrict__ src, int rows, int cols, uint8_t* __restrict__ dst,
                           float* __restrict__ scales) {
    __shared__ float s_red[8];
    const int cb = blockIdx.x, rb = blockIdx.y, mat = blockIdx.z;
    const int ncb = cols / 128, nrb = (rows + 127) / 128;
    const size_t base = (size_t)mat * rows * cols;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < 128 * 32; i += 256) {
        const int r = rb * 128 + i / 32, c = cb * 128 + (i % 32) * 4;
        if (r < rows) {
#pragma unroll
            for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(static_cast<float>(src[base + (size_t)r * cols + c + j])));
        }
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
    const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    for (int i = threadIdx.x; i < 128 * 32; i += 256) {
        const int r = rb * 128 + i / 32, c = cb * 128 + (i % 32) * 4;
        if (r < rows) {
            uint32_t packed = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                packed |= (uint32_t)__nv_cvt_float_to_fp8(static_cast<float>(src[base + (size_t)r * cols + c + j]) * inv,
                                                          __NV_SATFINITE, __NV_E4M3) << (8 * j);
            *reinterpret_cast<uint32_t*>(dst + base + (size_t)r * cols + c) = packed;
        }
    }
    if (threadIdx.x == 0) scales[((size_t)mat * nrb + rb) * ncb + cb] = scale;
}

// ---- host side ------------------------------------------------------------------------------------------------------
// (outer, rows, K) byte tensor, K contiguous; box = 128 bytes x box_rows x 1 with the 128-byte swizzle.
aristos_status_t make_map_u8(CUtensorMap* tm, const void* base, int K, int rows, int outer, int box_rows) {
    static_assert(F8_KB == 128, "one swizzle row per box row");
    return encode_map_3d(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, K, rows, outer, box_rows);
}

aristos_status_t launch_fp8_gemm(const void* A, const void* B0, const void* B1, const Fp8GemmParams& p,
                                 const Fp8PeerArgs& pa, int grid_limit, cudaStream_t st) {
    CUtensorMap tmA, tmB0, tmB1;
    ARISTOS_TRY(make_map_u8(&tmA, A, p.K, p.rows_per_group, p.groups, 128));
    ARISTOS_TRY(make_map_u8(&tmB0, B0, p.K, p.N, p.experts, 128));
    ARISTOS_TRY(make_map_u8(&tmB1, B1, p.K, p.N, p.experts, 128));
    // promotion warps per lane quarter: 2 (ARISTOS_FP8_PROMOTION_WARPS=4 selects four: measured slower, 2.31 ms
    // against 1.92 ms for 32 experts x 1024 rows, H 7168, I 2048 - 608 threads leave each 96 registers)
    static int subs = 0;
    if (subs == 0) {
        const char* env = getenv("ARISTOS_FP8_PROMOTION_WARPS");
        subs = (env && atoi(env) == 4) ? 4 : 2;
    }
    ARISTOS_CUDA_TRY(cudaFuncSetAttribute(ffn_fp8_grouped_gemm_kernel<2, false>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
    ARISTOS_CUDA_TRY(cudaFuncSetAttribute(ffn_fp8_grouped_gemm_kernel<2, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
    ARISTOS_CUDA_TRY(cudaFuncSetAttribute(ffn_fp8_grouped_gemm_kernel<4, false>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES));
    const int out_w = p.gated ? 128 : 256;
    int sms = device_sm_count();
    if (sms <= 0) { set_last_error("no CUDA device"); return ARISTOS_ERR_CUDA; }
    if (grid_limit > 0 && grid_limit < sms) sms = grid_limit;
    const int64_t bound = (int64_t)p.groups * ceil_div(p.row_end - p.row_begin, F8_BM) * ceil_div(p.N, out_w);
    const int grid = (int)(bound < sms ? bound : sms);
    if (grid <= 0) return ARISTOS_OK;
    if (p.outq) ffn_fp8_grouped_gemm_kernel<2, true><<<grid, f8_threads(2), F8_SMEM_BYTES, st>>>(tmA, tmB0, tmB1, p, pa);
    else if (subs == 2) ffn_fp8_grouped_gemm_kernel<2, false><<<grid, f8_threads(2), F8_SMEM_BYTES, st>>>(tmA, tmB0, tmB1, p, pa);
    else ffn_fp8_grouped_gemm_kernel<4, false><<<grid, f8_threads(4), F8_SMEM_BYTES, st>>>(tmA, tmB0, tmB1, p, pa);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace

// xq (groups, rows, H) e4m3 with sx (groups*rows, H/128); w1q/w3q (experts, I, H) with s1/s3 (experts, I/128, H/128);
// w2q (experts, H, I) with s2 (experts, H/128, I/128); h (bf16), hq + sh: scratch; y (groups, rows, H) bf16.
aristos_status_t expert_ffn_fp8_sm100(const void* xq, const float* sx, const int32_t* count, int groups,
                                      int rows_per_group, int experts, const void* w1q, const float* s1,
                                      const void* w3q, const float* s3, const void* w2q, const float* s2, void* h,
                                      void* hq, float* sh, void* y, int H, int I, int hidden_act, int row_begin,
                                      int row_end, int sm_limit, int32_t* dev_status, cudaStream_t st,
                                      void* const* peer_y, int peer_world, int peer_rank, const int32_t* dense_src_off,
                                      int dense_ret_rows) {
    const int want_groups = dense_src_off ? experts : peer_world * experts;
    if (peer_world > 8 || (peer_world > 0 && (!peer_y || groups != want_groups)) || (dense_src_off && peer_world == 0)) {
        set_last_error("expert_ffn(fp8): peer output needs world <= 8 and groups == world * experts (experts when dense)");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (groups > F8_MAX_GROUPS) { set_last_error("expert_ffn(fp8): more than %d row groups", F8_MAX_GROUPS); return ARISTOS_ERR_CONFIG; }
    if (H % 128 != 0 || I % 128 != 0) { set_last_error("expert_ffn(fp8): H and I must be multiples of 128"); return ARISTOS_ERR_CONFIG; }
    if (row_begin % F8_BM != 0) { set_last_error("expert_ffn(fp8): row_begin must be a multiple of 128"); return ARISTOS_ERR_INVALID_ARG; }
    const bool gated = hidden_act == ARISTOS_ACT_SWIGLU;
    Fp8GemmParams p{};
    p.count = count;
    p.groups = groups;
    p.experts = experts;
    p.rows_per_group = rows_per_group;
    p.row_begin = row_begin;
    p.row_end = row_end;
    p.dev_status = dev_status;
    p.N = I; p.K = H; p.gated = gated ? 1 : 0; p.act = hidden_act;
    p.sa = sx; p.sb0 = s1; p.sb1 = gated ? s3 : s1;
    p.out = static_cast<__nv_bfloat16*>(h);
    Fp8PeerArgs pa{};
    // ARISTOS_FP8_FUSED_QUANT=0: the up projection writes bf16 and a kernel of its own quantises it (the same bits)
    static int fused_quant = -1;
    if (fused_quant < 0) {
        const char* env = getenv("ARISTOS_FP8_FUSED_QUANT");
        fused_quant = (env && strcmp(env, "0") == 0) ? 0 : 1;
    }
    if (fused_quant) {
        // the up projection's epilogue quantises its own output rows: no bf16 copy of the hidden activations
        p.outq = static_cast<uint8_t*>(hq);
        p.out_scales = sh;
        ARISTOS_TRY(launch_fp8_gemm(xq, w1q, gated ? w3q : w1q, p, pa, sm_limit, st));
        p.outq = nullptr;
        p.out_scales = nullptr;
    } else {
        ARISTOS_TRY(launch_fp8_gemm(xq, w1q, gated ? w3q : w1q, p, pa, sm_limit, st));
        // hidden activations: bf16 -> e4m3 per row and 128 columns (valid rows only)
        quantize_group_rows_fp8_kernel<__nv_bfloat16><<<device_sm_count() * 4, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(h), count, groups, rows_per_group, I, static_cast<uint8_t*>(hq), sh);
        ARISTOS_COUNT_LAUNCH();
    }
    p.N = H; p.K = I; p.gated = 0; p.act = ARISTOS_ACT_IDENTITY;
    p.sa = sh; p.sb0 = s2; p.sb1 = s2;
    p.out = static_cast<__nv_bfloat16*>(y);
    pa.peer_world = peer_world;
    pa.peer_rank = peer_rank;
    pa.src_off = dense_src_off;
    pa.ret_rows = dense_ret_rows;
    for (int d = 0; d < peer_world; ++d) pa.peer_out[d] = static_cast<__nv_bfloat16*>(peer_y[d]);
    ARISTOS_TRY(launch_fp8_gemm(hq, w2q, w2q, p, pa, sm_limit, st));
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace aristos

using namespace aristos;

extern "C" aristos_status_t aristos_quantize_fp8(const void* src, int64_t mats, int64_t rows, int cols, int block_rows,
                                                 int src_dtype, void* dst_fp8, float* scales, void* stream) {
    if (!src || !dst_fp8 || !scales) { set_last_error("quantize_fp8: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (mats < 1 || rows < 0 || cols <= 0 || cols % 128 != 0 || (block_rows != 1 && block_rows != 128)) {
        set_last_error("quantize_fp8: cols must be a multiple of 128 and block_rows 1 or 128");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (src_dtype != ARISTOS_DTYPE_BF16 && src_dtype != ARISTOS_DTYPE_F32) {
        set_last_error("quantize_fp8: source dtype must be bf16 or fp32");
        return ARISTOS_ERR_UNSUPPORTED;
    }
    if (rows == 0) return ARISTOS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (block_rows == 1) {
        const int64_t all = mats * rows;
        int64_t blocks = (all * (cols / 128) * 32 + 255) / 256;
        const int64_t cap_blocks = (int64_t)device_sm_count() * 8;
        if (blocks > cap_blocks) blocks = cap_blocks;
        if (src_dtype == ARISTOS_DTYPE_BF16)
            quantize_rows_fp8_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
                (const __nv_bfloat16*)src, all, cols, (uint8_t*)dst_fp8, scales);
        else
            quantize_rows_fp8_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)src, all, cols,
                                                                              (uint8_t*)dst_fp8, scales);
    } else {
        if (mats > 65535 || (rows + 127) / 128 > 65535) { set_last_error("quantize_fp8: tensor too large"); return ARISTOS_ERR_CONFIG; }
        dim3 grid(cols / 128, (unsigned)((rows + 127) / 128), (unsigned)mats);
        if (src_dtype == ARISTOS_DTYPE_BF16)
            quantize_blocks_fp8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, (int)rows, cols,
                                                                            (uint8_t*)dst_fp8, scales);
        else
            quantize_blocks_fp8_kernel<float><<<grid, 256, 0, st>>>((const float*)src, (int)rows, cols, (uint8_t*)dst_fp8,
                                                                    scales);
    }
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}
