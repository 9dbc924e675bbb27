// Gate: logits = x * Wg^T (+ bias) in fp32 with a fixed reduction order, top-k on the logits, softmax / sigmoid
// combine weights.
//
// The reference has no gate (its only trace is the unused gateScratch array, benchmarks.cuh:168-178); operand
// layout follows its expert-tile contract: x (S,H) row-major, Wg (E,H) row-major = the (N,K) B operand of
// mma.cuh:396-397.
//
// Bit-exact contract (mirrored by the CPU oracle): for a token t and expert e there are 32 x 2 partial sums;
//   p[c][h % 2] = fmaf(x[t,h], Wg[e,h], p[c][h % 2])   over the 8-element chunks q = h/8 with q % 32 == c, in
// increasing h (even and odd elements accumulate separately, so fp32 rows take one packed two-lane FMA per pair), then
// P[c] = p[c][0] + p[c][1], the 32 values P[c] are combined by the xor butterfly 16, 8, 4, 2, 1
// (P[c] = P[c] + P[c ^ m]) and the bias is added last. Products of bf16 values are exact in fp32 and every step is
// one IEEE operation, so the logits do not depend on the launch geometry and the CPU reproduces them bit for bit.
// Top-k is taken on the logits (exp is monotone, so the selected indices cannot depend on its rounding); ties go to
// the lower expert index.
//
// Kernel shape: a CTA of 16 warps owns a tile of tokens x experts; H is walked in slabs of 256 elements that are
// staged in shared memory with cp.async (three stages), lane c of every warp reads chunk c of a slab row, so lane c
// holds the partial sums c of its warp's 4-token x 8-expert register tile. fp32 rows use packed fp32x2 FMAs (half the
// issue slots of scalar FMAs); bf16 / fp16 rows use the mixed-precision FMA on the raw 16-bit operands (fp32
// accumulator, one rounding: the same bits as converting first), so nothing is unpacked on the integer pipe.
// The butterfly is done as a reduce-scatter
// (each step keeps half of the tile, 31 shuffles instead of 160): adding the same two operands, it gives the same
// bits as the full butterfly. With few experts the kernel streams x once from HBM; with many it is FMA-bound.
#include "common.cuh"
#include "gate_contract.cuh"

namespace aristos {

constexpr int GATE_THREADS = 512;
constexpr int GATE_WARPS = GATE_THREADS / 32;
constexpr int GATE_TT = 4;       // tokens per warp register tile
constexpr int GATE_TE = 8;       // experts per warp register tile
constexpr int GATE_SLAB = 256;   // elements of H per staged slab (one 8-element chunk per lane)

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int GATE_STAGES = 3;

// Top-k on one token's logits (in shared memory) by one warp, then the combine weights.
__device__ __forceinline__ void topk_one_token(const float* l, int t, int E, int k, int gate_fn, int renorm, int lane,
                                               int32_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                                               float* __restrict__ logits_out) {
    if (logits_out)
        for (int e = lane; e < E; e += 32) logits_out[(size_t)t * E + e] = l[e];
    int chosen[MAX_TOPK];
    float chosen_l[MAX_TOPK];
#pragma unroll 1
    for (int j = 0; j < k; ++j) {
        float bv = 0.0f;
        int bi = -1;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int i = 0; i < j; ++i) taken |= (chosen[i] == e);
            if (taken) continue;
            const float v = l[e];
            if (bi < 0 || v > bv) { bv = v; bi = e; }   // strict '>' keeps the lowest index within a lane
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
            const bool take = (oi >= 0) && (bi < 0 || ov > bv || (ov == bv && oi < bi));
            if (take) { bv = ov; bi = oi; }
        }
        chosen[j] = bi;
        chosen_l[j] = bv;
    }
    float w_sel[MAX_TOPK];
    if (gate_fn == ARISTOS_GATE_SOFTMAX) {
        const float mx = chosen_l[0];
        float den = 0.0f;
        for (int e = lane; e < E; e += 32) den += expf(l[e] - mx);
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) den += __shfl_xor_sync(0xffffffffu, den, m);
        for (int j = 0; j < k; ++j) w_sel[j] = expf(chosen_l[j] - mx) / den;
    } else {
        for (int j = 0; j < k; ++j) w_sel[j] = 1.0f / (1.0f + expf(-chosen_l[j]));
    }
    if (renorm) {
        float s = 0.0f;
        for (int j = 0; j < k; ++j) s += w_sel[j];
        for (int j = 0; j < k; ++j) w_sel[j] = w_sel[j] / s;
    }
    for (int j = 0; j < k; ++j)
        if (lane == j) {
            topk_idx[(size_t)t * k + j] = chosen[j];
            topk_w[(size_t)t * k + j] = w_sel[j];
        }
}

// xor butterfly 16, 8, 4, 2, 1 over the lanes as a reduce-scatter of a 4 x 8 register tile: each step keeps half of
// the tile; afterwards a[0] of lane c is the fully reduced tile element c (token c >> 3, expert c & 7).
__device__ __forceinline__ float reduce_scatter_tile(float (&a)[GATE_TT * GATE_TE], int lane) {
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
        const bool up = (lane & half) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float keep = up ? a[i + half] : a[i];
            const float send = up ? a[i] : a[i + half];
            a[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
        }
    }
    return a[0];
}

// Few experts (E <= 8): every warp streams its own 4 token rows (Wg stays in L1) with no block-wide barrier; same
// arithmetic, same bits. The rows arrive through a per-lane ring in shared memory filled by cp.async three slabs
// ahead: each lane reads back only the 16 bytes it copied itself, so the ring needs no synchronisation at all, and
// the loads in flight do not cost registers (the 4 x 8 accumulator tile already takes 64).
constexpr int STREAM_WARPS = 8;
constexpr int STREAM_STAGES = 4;
constexpr int STREAM_SMEM_BYTES = STREAM_WARPS * STREAM_STAGES * GATE_TT * 32 * 16;
template <typename T>
__global__ void __launch_bounds__(STREAM_WARPS * 32)
gate_topk_stream_kernel(const T* __restrict__ x, const T* __restrict__ wg, const float* __restrict__ bias, int S, int H,
                        int E, int k, int gate_fn, int renorm, int32_t* __restrict__ topk_idx,
                        float* __restrict__ topk_w, float* __restrict__ logits_out) {
    constexpr int PIECES = (int)sizeof(T) / 2;            // 16-byte pieces per 8-element chunk (fp32: 2)
    extern __shared__ __align__(16) uint8_t stream_smem[];
    __shared__ float s_logits[STREAM_WARPS][GATE_TT][GATE_TE];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = (blockIdx.x * STREAM_WARPS + warp) * GATE_TT;
    if (t0 >= S) return;
    const int nchunk = H >> 3;
    const int nslab = (nchunk + 31) >> 5;
    const T* xrow[GATE_TT];
    const T* wrow[GATE_TE];
#pragma unroll
    for (int tt = 0; tt < GATE_TT; ++tt) xrow[tt] = x + (size_t)min(t0 + tt, S - 1) * H;
#pragma unroll
    for (int ee = 0; ee < GATE_TE; ++ee) wrow[ee] = wg + (size_t)min(ee, E - 1) * H;
    // ring entry (stage, token, lane): 16 bytes
    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(stream_smem)) +
                          (uint32_t)warp * (STREAM_STAGES * GATE_TT * 512) + lane * 16;
    const uint8_t* ring_ptr = stream_smem + warp * (STREAM_STAGES * GATE_TT * 512) + lane * 16;
    auto issue = [&](int slab) {
        // chunk slab*32 + lane of every row (16-bit rows: one 16-byte piece)
        const int piece = slab * 32 + lane;
        if (slab < nslab && piece < nchunk) {
#pragma unroll
            for (int tt = 0; tt < GATE_TT; ++tt)
                cp_async_16(ring + ((slab % STREAM_STAGES) * GATE_TT + tt) * 512,
                            reinterpret_cast<const uint8_t*>(xrow[tt]) + (size_t)piece * 16, 16);
        }
        cp_async_commit();
    };
    float2 acc[GATE_TT][GATE_TE];
#pragma unroll
    for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
        for (int ee = 0; ee < GATE_TE; ++ee) acc[tt][ee] = make_float2(0.0f, 0.0f);
    if (PIECES == 1) {
        // 16-bit rows: lane c owns the chunks q % 32 == c
#pragma unroll
        for (int s = 0; s < STREAM_STAGES - 1; ++s) issue(s);
        for (int slab = 0; slab < nslab; ++slab) {
            cp_async_wait<STREAM_STAGES - 2>();
            issue(slab + STREAM_STAGES - 1);
            const int q = slab * 32 + lane;
            if (q < nchunk) {
                GateChunk<T> xv[GATE_TT];
#pragma unroll
                for (int tt = 0; tt < GATE_TT; ++tt)
                    load_chunk(reinterpret_cast<const T*>(ring_ptr + ((slab % STREAM_STAGES) * GATE_TT + tt) * 512), xv[tt]);
#pragma unroll
                for (int ee = 0; ee < GATE_TE; ++ee) {
                    GateChunk<T> wv;
                    load_chunk(wrow[ee] + q * 8, wv);
#pragma unroll
                    for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) fma_pair(acc[tt][ee], xv[tt], wv, i);
                }
            }
        }
    } else {
        // fp32 rows: straight from global memory (the fp32 gate is the small reference case)
        for (int q = lane; q < nchunk; q += 32) {
            GateChunk<T> xv[GATE_TT];
#pragma unroll
            for (int tt = 0; tt < GATE_TT; ++tt) load_chunk(xrow[tt] + q * 8, xv[tt]);
#pragma unroll
            for (int ee = 0; ee < GATE_TE; ++ee) {
                GateChunk<T> wv;
                load_chunk(wrow[ee] + q * 8, wv);
#pragma unroll
                for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) fma_pair(acc[tt][ee], xv[tt], wv, i);
            }
        }
    }
    float a[GATE_TT * GATE_TE];
#pragma unroll
    for (int i = 0; i < GATE_TT * GATE_TE; ++i) a[i] = acc[i / GATE_TE][i % GATE_TE].x + acc[i / GATE_TE][i % GATE_TE].y;
    float p = reduce_scatter_tile(a, lane);
    {
        const int tt = lane >> 3, ee = lane & 7;
        if (ee < E) {
            if (bias) p = p + bias[ee];
            s_logits[warp][tt][ee] = p;
        }
    }
    __syncwarp();
    for (int tt = 0; tt < GATE_TT; ++tt) {
        const int t = t0 + tt;
        if (t >= S) break;
        topk_one_token(&s_logits[warp][tt][0], t, E, k, gate_fn, renorm, lane, topk_idx, topk_w, logits_out);
    }
}


// WT x WE warps: the CTA tile is (WT*4) tokens x (WE*8) experts; experts beyond that are walked in further tiles.
template <typename T, int WT, int WE>
__global__ void __launch_bounds__(GATE_THREADS)
gate_topk_kernel(const T* __restrict__ x, const T* __restrict__ wg, const float* __restrict__ bias, int S, int H,
                 int E, int k, int gate_fn, int renorm, int32_t* __restrict__ topk_idx,
                 float* __restrict__ topk_w, float* __restrict__ logits_out) {
    static_assert(WT * WE == GATE_WARPS, "warp grid");
    constexpr int TOK = WT * GATE_TT, ET = WE * GATE_TE, ROWS = TOK + ET;
    constexpr int ROW_BYTES = GATE_SLAB * (int)sizeof(T);
    constexpr int CHUNKS16 = ROW_BYTES / 16 / 32;            // 16-byte pieces per lane and row (1 for bf16, 2 for fp32)
    extern __shared__ __align__(16) uint8_t gate_smem[];
    uint8_t* stage_mem = gate_smem;                          // [GATE_STAGES][ROWS][ROW_BYTES]
    float* s_logits = reinterpret_cast<float*>(gate_smem + GATE_STAGES * ROWS * ROW_BYTES);   // [TOK][E]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wt = warp / WE, we = warp % WE;
    const int t0 = blockIdx.x * TOK;
    const int nchunk = H >> 3;
    const int nslab = (nchunk + 31) >> 5;
    const int etiles = (E + ET - 1) / ET;
    const uint32_t stage_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(stage_mem));

    // one slab of one expert tile: rows 0..TOK-1 = tokens, TOK..ROWS-1 = experts; invalid pieces are zero-filled
    auto issue_slab = [&](int etile, int slab, int buf) {
        for (int r = warp; r < ROWS; r += GATE_WARPS) {
            const bool is_tok = r < TOK;
            const int row = is_tok ? t0 + r : etile * ET + (r - TOK);
            const bool row_ok = is_tok ? (row < S) : (row < E);
            const T* base = (is_tok ? x : wg) + (size_t)(row_ok ? row : 0) * H;
#pragma unroll
            for (int u = 0; u < CHUNKS16; ++u) {
                // lane's 8-element chunk of this slab is q = slab*32 + lane; it spans CHUNKS16 16-byte pieces
                const int q = slab * 32 + lane;
                const bool ok = row_ok && q < nchunk;
                const uint8_t* src = reinterpret_cast<const uint8_t*>(base + (size_t)(ok ? q : 0) * 8) + u * 16;
                const uint32_t dst = stage_u32 + (buf * ROWS + r) * ROW_BYTES + lane * (16 * CHUNKS16) + u * 16;
                cp_async_16(dst, src, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };

    for (int etile = 0; etile < etiles; ++etile) {
        float2 acc[GATE_TT][GATE_TE];      // (even, odd) partial sums
#pragma unroll
        for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
            for (int ee = 0; ee < GATE_TE; ++ee) acc[tt][ee] = make_float2(0.0f, 0.0f);

        // three-stage pipeline, one barrier per slab: slab s lives in buffer s % 3
        issue_slab(etile, 0, 0);
        if (nslab > 1) issue_slab(etile, 1, 1); else cp_async_commit();
        for (int slab = 0; slab < nslab; ++slab) {
            cp_async_wait<1>();            // all groups but the newest have landed: slab `slab` is in shared memory
            __syncthreads();               // ... for every thread, and buffer (slab + 2) % 3 is no longer being read
            if (slab + 2 < nslab) issue_slab(etile, slab + 2, (slab + 2) % GATE_STAGES); else cp_async_commit();
            const T* srow = reinterpret_cast<const T*>(stage_mem + (size_t)(slab % GATE_STAGES) * ROWS * ROW_BYTES);
            GateChunk<T> xv[GATE_TT];
#pragma unroll
            for (int tt = 0; tt < GATE_TT; ++tt) load_chunk(srow + (wt * GATE_TT + tt) * GATE_SLAB + lane * 8, xv[tt]);
#pragma unroll
            for (int ee = 0; ee < GATE_TE; ++ee) {
                GateChunk<T> wv;
                load_chunk(srow + (TOK + we * GATE_TE + ee) * GATE_SLAB + lane * 8, wv);
#pragma unroll
                for (int tt = 0; tt < GATE_TT; ++tt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) fma_pair(acc[tt][ee], xv[tt], wv, i);
            }
        }
        __syncthreads();                   // the next expert tile restarts the pipeline in buffers 0 and 1

        float a[GATE_TT * GATE_TE];
#pragma unroll
        for (int i = 0; i < GATE_TT * GATE_TE; ++i) a[i] = acc[i / GATE_TE][i % GATE_TE].x + acc[i / GATE_TE][i % GATE_TE].y;
        const float tile_elem = reduce_scatter_tile(a, lane);
        {
            const int tt = lane >> 3, ee = lane & 7;
            const int e = etile * ET + we * GATE_TE + ee;
            if (e < E) {
                float p = tile_elem;
                if (bias) p = p + bias[e];
                s_logits[(wt * GATE_TT + tt) * E + e] = p;
            }
        }
    }
    __syncthreads();

    // ---- top-k and weights: one warp per token -------------------------------------------------------------------
    for (int tl = warp; tl < TOK; tl += GATE_WARPS) {
        const int t = t0 + tl;
        if (t >= S) break;
        topk_one_token(s_logits + tl * E, t, E, k, gate_fn, renorm, lane, topk_idx, topk_w, logits_out);
    }
}

template <typename T, int WT, int WE>
static aristos_status_t launch_gate_shape(const void* x, const void* wg, const float* bias, int S, int H, int E, int k,
                                          int gate_fn, int renorm, int32_t* topk_idx, float* topk_w,
                                          float* logits_out, cudaStream_t stream) {
    constexpr int TOK = WT * GATE_TT, ET = WE * GATE_TE, ROWS = TOK + ET;
    const size_t smem = GATE_STAGES * (size_t)ROWS * GATE_SLAB * sizeof(T) + sizeof(float) * (size_t)TOK * E;
    auto kernel = gate_topk_kernel<T, WT, WE>;
    if (smem > 48 * 1024)
        ARISTOS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = ceil_div(S, TOK);
    kernel<<<grid, GATE_THREADS, smem, stream>>>(static_cast<const T*>(x), static_cast<const T*>(wg), bias, S, H, E, k,
                                                 gate_fn, renorm, topk_idx, topk_w, logits_out);
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

template <typename T>
static aristos_status_t launch_gate(const void* x, const void* wg, const float* bias, int S, int H, int E, int k,
                                    int gate_fn, int renorm, int32_t* topk_idx, float* topk_w, float* logits_out,
                                    cudaStream_t stream) {
    // few experts: wide token tiles (x streams once from HBM); many experts: 32-expert tiles walked per CTA
    if (E <= 8) {
        const int grid = ceil_div(S, STREAM_WARPS * GATE_TT);
        ARISTOS_CUDA_TRY(cudaFuncSetAttribute(gate_topk_stream_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              STREAM_SMEM_BYTES));
        gate_topk_stream_kernel<T><<<grid, STREAM_WARPS * 32, STREAM_SMEM_BYTES, stream>>>(
            static_cast<const T*>(x), static_cast<const T*>(wg), bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w,
            logits_out);
        ARISTOS_COUNT_LAUNCH();
        ARISTOS_CUDA_TRY(cudaGetLastError());
        return ARISTOS_OK;
    }
    if (E <= 16)
        return launch_gate_shape<T, 8, 2>(x, wg, bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, stream);
    if (E <= 32)
        return launch_gate_shape<T, 4, 4>(x, wg, bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, stream);
    // 8 tokens x 64 experts per CTA: small token tiles keep the last wave of CTAs full
    return launch_gate_shape<T, 2, 8>(x, wg, bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, stream);
}

}  // namespace aristos

using namespace aristos;

extern "C" aristos_status_t aristos_gate_topk(const void* x, const void* w_gate, const float* gate_bias, int S,
                                              int H, int E, int k, int gate_fn, int renorm, int dtype,
                                              int32_t* topk_idx, float* topk_w, float* logits_out, void* stream) {
    if (!x || !w_gate || !topk_idx || !topk_w) { set_last_error("gate: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (S < 0 || H <= 0 || E <= 0 || k <= 0) { set_last_error("gate: bad size"); return ARISTOS_ERR_INVALID_ARG; }
    if (H % 8 != 0 || k > E || k > MAX_TOPK || E > 1024) {
        set_last_error("gate: need H %% 8 == 0, k <= min(E, %d), E <= 1024", MAX_TOPK);
        return ARISTOS_ERR_CONFIG;
    }
    if (!aligned16(x) || !aligned16(w_gate)) { set_last_error("gate: pointers must be 16-byte aligned"); return ARISTOS_ERR_INVALID_ARG; }
    if (gate_fn != ARISTOS_GATE_SOFTMAX && gate_fn != ARISTOS_GATE_SIGMOID) return ARISTOS_ERR_INVALID_ARG;
    if (S == 0) return ARISTOS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ARISTOS_DTYPE_F32:
        case ARISTOS_DTYPE_TF32:
            return launch_gate<float>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, st);
        case ARISTOS_DTYPE_BF16:
            return launch_gate<__nv_bfloat16>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, st);
        case ARISTOS_DTYPE_F16:
            return launch_gate<__half>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, logits_out, st);
        default:
            set_last_error("gate: dtype %d not implemented (f32, bf16 and f16 are)", dtype);
            return ARISTOS_ERR_UNSUPPORTED;
    }
}
