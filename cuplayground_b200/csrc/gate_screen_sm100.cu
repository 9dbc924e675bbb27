// Gate for many experts: a tensor-core screen followed by exact evaluation of the experts that can still win.
//
// The routing must follow the bit-exact logit contract of gate.cu (fixed-order fp32 FMAs), which keeps the full
// S x E x H product off the tensor cores: their accumulation order is not specified. But top-k only needs the exact
// logits of experts close to the k-th place. So:
//   1. gate_wnorm_kernel   : |Wg[e,:]|_2 per expert.
//   2. gate_screen_kernel  : approximate logits A = x * Wg^T with tcgen05.mma (fp32 accumulators in TMEM, operands by
//                            TMA). H is cut into slices of 512 elements; each slice's partial sums start from zero
//                            and go to scratch on their own, which keeps the accumulation chains short.
//   3. gate_select_kernel  : one warp per token. With err[e] >= |A[e] - L[e]| (L = the contract's logit), every expert
//                            whose upper bound A[e] + err[e] reaches the k-th largest lower bound A[e] - err[e] is a
//                            candidate; no other expert can be among the top k. The candidates' logits are computed
//                            exactly as in gate.cu, top-k (ties -> lower index) runs on those, and the softmax
//                            denominator takes exact logits for candidates and screened ones for the rest.
// err[e] = 4 n 2^-23 |x_t| |Wg_e| + (slices) 2^-24 sum|slice sums| + 2^-20 max|A|, n = elements per slice. Products of
// 16-bit inputs are exact, so A and L differ from the true dot product only by accumulation roundings. Inside a slice,
// n accumulations that each lose at most one unit in the last place of a partial sum bounded by sum|x_h w_h| give
// n 2^-23 sum|x_h w_h|; over the slices, sum_s |x_s||w_s| <= |x||w| (Cauchy-Schwarz, twice). The factor 4 covers
// block-wise alignment and truncation inside the tensor core and the contract's own roundings. The second term is the
// fp32 sum over the slices (computed from the values added), the third the bias addition. The select kernel also
// checks the bound on every candidate (where it has both values) and on one expert that the screen ruled out (the one
// whose upper bound came closest to the k-th place: what a bound that is too small would drop first); a token that
// violates it is evaluated exactly over all experts and DEV_FAULT_SCREEN is raised in the status word - an error, not
// a warning, because a bound that fails where it is checked cannot be trusted where it is not. Tokens whose logits are
// NaN leave no candidate: they raise DEV_FAULT_NONFINITE instead.
// The routing is therefore identical to gate.cu's; only the weights of a softmax gate may differ in the last bits
// (the screened logits of non-candidates enter the denominator). Used by the layer when no logits are requested,
// for 16-bit inputs and many experts (up to 256).
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "gate_contract.cuh"
#include "ptx_sm100.cuh"
#include "tensor_map.cuh"

namespace aristos {

namespace {

constexpr int GS_BM = 128;                      // tokens per tile
constexpr int GS_BK = 64;                       // 128 bytes of K per stage row
constexpr int GS_STAGES = 4;
constexpr int GS_THREADS = 192;                 // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int GS_A_BYTES = GS_BM * GS_BK * 2;   // 16 KB
constexpr int GS_B_BOX_BYTES = 128 * GS_BK * 2; // one 128-expert box
constexpr int GS_STAGE_BYTES = GS_A_BYTES + 2 * GS_B_BOX_BYTES;
constexpr int GS_SMEM_BYTES = 1024 + GS_STAGES * GS_STAGE_BYTES + 256;
constexpr int GS_MAX_E = 256;
constexpr int GS_MAX_SLICES = 16;             // slices of H whose partial logits are stored separately
constexpr int GS_SLICE_KB = 8;                 // K blocks (of 64 elements) per slice, unless that needs more slices

struct GateScreenParams {
    int S, H, E;
    int n_mma;          // E rounded up to a multiple of 16
    int buf_cols;       // TMEM columns per accumulator buffer: power of two >= max(32, n_mma)
    int kblocks;        // ceil(H / 64)
    int slice_kb;       // K blocks per slice; every slice restarts the accumulator and is stored on its own
    int nslices;
    int bf16;           // 1: bf16 operands, 0: fp16
    float* partial;     // (nslices, S, E)
    int32_t* dev_status;
};

// CTA (x, y) owns the 128-token tile x and the slices y, y + gridDim.y, ... of H. Accumulators alternate between two
// TMEM buffers so that the stores of one slice run under the MMAs of the next.
__global__ void __launch_bounds__(GS_THREADS, 1)
gate_screen_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const GateScreenParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* aux = smem + GS_STAGES * GS_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(aux);             // full[S], empty[S], tfull[2], tempty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aux + 132);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = ptx::smem_u32(bars);
    const uint32_t bar_empty = bar_full + 8 * GS_STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * GS_STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t smem_base = ptx::smem_u32(smem);
    const int m0 = blockIdx.x * GS_BM;
    const int nbox = p.E > 128 ? 2 : 1;
    const uint32_t stage_tx = GS_A_BYTES + nbox * GS_B_BOX_BYTES;
    const uint32_t tmem_cols = 2 * p.buf_cols;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GS_STAGES; ++s) {
            ptx::mbar_init(bar_full + 8 * s, 1);
            ptx::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar_tfull + 8 * b, 1);
            ptx::mbar_init(bar_tempty + 8 * b, 128);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) ptx::tmem_alloc(ptx::smem_u32(tmem_slot), tmem_cols);
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmX);
            ptx::prefetch_tensormap(&tmW);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int sl = blockIdx.y; ok && sl < p.nslices; sl += gridDim.y) {
                const int kb0 = sl * p.slice_kb, kb1 = min(p.kblocks, kb0 + p.slice_kb);
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.dev_status);
                    if (!ok) break;
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * GS_STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(full, stage_tx);
                    ptx::tma_load_3d(sa, &tmX, kb * GS_BK, m0, 0, full);
                    for (int b = 0; b < nbox; ++b)
                        ptx::tma_load_3d(sa + GS_A_BYTES + b * GS_B_BOX_BYTES, &tmW, kb * GS_BK, b * 128, 0, full);
                    if (++stage == GS_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            const uint32_t idesc = ptx::umma_idesc_f32acc(GS_BM, p.n_mma, p.bf16 ? 1u : 0u);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int sl = blockIdx.y; ok && sl < p.nslices; sl += gridDim.y, ++it) {
                const int buf = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ok = ptx::mbar_wait_bounded(bar_tempty + 8 * buf, aphase ^ 1u, abort_flag, p.dev_status);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * p.buf_cols;
                const int kb0 = sl * p.slice_kb, kb1 = min(p.kblocks, kb0 + p.slice_kb);
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = ptx::mbar_wait_bounded(bar_full + 8 * stage, phase, abort_flag, p.dev_status);
                    if (!ok) break;
                    ptx::tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * GS_STAGE_BYTES;
                    const uint64_t da = ptx::umma_desc_k_sw128(sa);
                    const uint64_t db = ptx::umma_desc_k_sw128(sa + GS_A_BYTES);
#pragma unroll
                    for (int k = 0; k < GS_BK / 16; ++k)
                        ptx::umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    ptx::umma_commit(bar_empty + 8 * stage);
                    if (++stage == GS_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(bar_tfull + 8 * buf);
            }
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;                 // TMEM lanes this warp may read
        const int row = m0 + quarter * 32 + lane;
        int it = 0;
        for (int sl = blockIdx.y; sl < p.nslices; sl += gridDim.y, ++it) {
            const int buf = it & 1;
            const uint32_t aphase = (it >> 1) & 1u;
            // tcgen05.ld is warp-collective: the warp leaves together
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(bar_tfull + 8 * buf, aphase, abort_flag, p.dev_status)))
                break;
            ptx::tcgen05_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * p.buf_cols;
            float* out = p.partial + ((size_t)sl * p.S + (size_t)min(row, p.S - 1)) * p.E;
            for (int c0 = 0; c0 < p.n_mma; c0 += 32) {
                uint32_t a[32];
                ptx::tmem_ld_32x32b_x32(taddr + c0, a);
                ptx::tmem_ld_wait();
                if (c0 + 32 >= p.n_mma) {             // the last load has landed: hand the buffer back
                    ptx::tcgen05_fence_before();
                    ptx::mbar_arrive(bar_tempty + 8 * buf);
                }
                if (row < p.S) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (c0 + 4 * q < p.E)        // E is a multiple of 4
                            *reinterpret_cast<uint4*>(out + c0 + 4 * q) = make_uint4(a[4 * q], a[4 * q + 1], a[4 * q + 2], a[4 * q + 3]);
                }
            }
        }
    }

    ptx::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, tmem_cols);
    }
}

// |Wg[e,:]|_2 per expert, rounded up a little; one warp per expert.
template <typename T>
__global__ void __launch_bounds__(256) gate_wnorm_kernel(const T* __restrict__ wg, int E, int H, float* __restrict__ wnorm) {
    const int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (e >= E) return;
    float s = 0.0f;
    for (int q = lane; q < (H >> 3); q += 32) {
        float2 v[4];
        load8_pairs(wg + (size_t)e * H + q * 8, v);
#pragma unroll
        for (int i = 0; i < 4; ++i) s = fmaf(v[i].y, v[i].y, fmaf(v[i].x, v[i].x, s));
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (lane == 0) wnorm[e] = sqrtf(s) * 1.0001f;
}

constexpr int SEL_WARPS = 8;

// fp32 -> unsigned key with the same order (-0 and +0 compare equal, as they do as floats); 0 marks "removed".
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t u = __float_as_uint(v + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// The contract's logits of the experts cand[c0 .. c0+G) for one token, by one warp: lane c owns the chunks q % 32 == c,
// (even, odd) partial sums, P = even + odd, xor butterfly 16..1 (both partners add the same two values, so every lane
// ends with the same bits), bias last. G independent FMA chains per lane.
template <typename T, int G, int UNROLL>
__device__ __forceinline__ void exact_logits(const T* __restrict__ xrow, const T* __restrict__ wg,
                                             const float* __restrict__ bias, int H, const int* cand, int c0,
                                             float* exact, int lane) {
    const int nchunk = H >> 3;
    const T* wr[G];
    int ex[G];
    float2 acc[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
        ex[j] = cand[c0 + j];
        wr[j] = wg + (size_t)ex[j] * H;
        acc[j] = make_float2(0.0f, 0.0f);
    }
#pragma unroll UNROLL
    for (int q = lane; q < nchunk; q += 32) {
        GateChunk<T> xv;
        load_chunk(xrow + q * 8, xv);
#pragma unroll
        for (int j = 0; j < G; ++j) {
            GateChunk<T> wv;
            load_chunk(wr[j] + q * 8, wv);
#pragma unroll
            for (int i = 0; i < 4; ++i) fma_pair(acc[j], xv, wv, i);
        }
    }
#pragma unroll
    for (int j = 0; j < G; ++j) {
        float P = acc[j].x + acc[j].y;
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) P = P + __shfl_xor_sync(0xffffffffu, P, m);
        if (bias) P = P + bias[ex[j]];
        if (lane == j) exact[c0 + j] = P;
    }
}

template <typename T>
__device__ __forceinline__ void exact_logits_all(const T* __restrict__ xrow, const T* __restrict__ wg,
                                                 const float* __restrict__ bias, int H, const int* cand, int n,
                                                 float* exact, int lane) {
    int c0 = 0;
    for (; c0 + 4 <= n; c0 += 4) exact_logits<T, 4, 2>(xrow, wg, bias, H, cand, c0, exact, lane);
    if (n - c0 >= 2) { exact_logits<T, 2, 4>(xrow, wg, bias, H, cand, c0, exact, lane); c0 += 2; }
    if (n - c0 >= 1) exact_logits<T, 1, 4>(xrow, wg, bias, H, cand, c0, exact, lane);
    __syncwarp();
}

// SLOTS experts per lane: e = lane + 32 * slot.
template <typename T, int SLOTS>
__global__ void __launch_bounds__(SEL_WARPS * 32)
gate_select_kernel(const T* __restrict__ x, const T* __restrict__ wg, const float* __restrict__ bias,
                   const float* __restrict__ partial, int nslices, const float* __restrict__ wnorm, int S, int H, int E,
                   int k, int gate_fn, int renorm, float err_scale, int32_t* __restrict__ topk_idx,
                   float* __restrict__ topk_w, int32_t* dev_status) {
    __shared__ int s_cand[SEL_WARPS][SLOTS * 32];
    __shared__ float s_exact[SEL_WARPS][SLOTS * 32];
    __shared__ uint32_t s_key[SEL_WARPS][SLOTS * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * SEL_WARPS + warp;
    if (t >= S) return;
    int* cand = s_cand[warp];
    float* exact = s_exact[warp];
    uint32_t* ekey = s_key[warp];
    const T* xrow = x + (size_t)t * H;
    const float NEG_INF = __int_as_float(0xff800000);

    // screened logits (the slices' partial sums added in a fixed order), |x_t|, error bounds
    float a[SLOTS], err[SLOTS];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        const int e = lane + 32 * i;
        a[i] = NEG_INF;
        err[i] = 0.0f;
        if (e < E) {
            float v = 0.0f, vabs = 0.0f;
            for (int s = 0; s < nslices; ++s) {
                const float ps = partial[((size_t)s * S + t) * E + e];
                v += ps;
                vabs += fabsf(ps);
            }
            if (bias) v += bias[e];
            a[i] = v;
            err[i] = (float)nslices * 5.9604644775390625e-8f * vabs * 1.0001f;   // the fp32 sum over the slices
            amax = fmaxf(amax, fabsf(v));
        }
    }
    float2 nx2 = make_float2(0.0f, 0.0f);
    for (int q = lane; q < (H >> 3); q += 32) {
        GateChunk<T> xv;
        load_chunk(xrow + q * 8, xv);
#pragma unroll
        for (int i = 0; i < 4; ++i) fma_pair(nx2, xv, xv, i);
    }
    float nx = nx2.x + nx2.y;
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
        nx += __shfl_xor_sync(0xffffffffu, nx, m);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    }
    nx = sqrtf(nx) * 1.0001f;

    // k-th largest lower bound A - err, in key space
    uint32_t lk[SLOTS];
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        const int e = lane + 32 * i;
        err[i] = e < E ? err[i] + err_scale * nx * wnorm[e] + 9.5367431640625e-7f * amax : 0.0f;
        lk[i] = e < E ? order_key(a[i] - err[i]) : 0u;
    }
    uint32_t kth = 0u;
#pragma unroll 1
    for (int j = 0; j < k; ++j) {
        uint32_t bk = 0u;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) bk = max(bk, lk[i]);
        kth = __reduce_max_sync(0xffffffffu, bk);
        const uint32_t owners = __ballot_sync(0xffffffffu, bk == kth);
        if (lane == __ffs(owners) - 1) {               // one holder of the maximum drops one instance of it
            bool done = false;
#pragma unroll
            for (int i = 0; i < SLOTS; ++i)
                if (!done && lk[i] == kth) { lk[i] = 0u; done = true; }
        }
    }

    // candidates: upper bound reaches the k-th lower bound (ascending expert index along the list)
    int n = 0;
    int pos[SLOTS];
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        const int e = lane + 32 * i;
        const bool pred = e < E && order_key(a[i] + err[i]) >= kth;
        const uint32_t mask = __ballot_sync(0xffffffffu, pred);
        pos[i] = pred ? n + __popc(mask & ((1u << lane) - 1u)) : -1;
        if (pred) cand[pos[i]] = e;
        n += __popc(mask);
    }
    // One expert that the screen ruled out is evaluated exactly all the same: the one whose upper bound came closest
    // to the k-th place. It is the likeliest victim of an error bound that does not hold, and no candidate check
    // would ever see it. It sits behind the candidates in the list (entry n) and takes no part in the top-k.
    int probe_slot = -1;         // slot of the probed expert in the lane that owns it
    {
        uint32_t bk = 0u;
        int bs = -1;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) {
            const int e = lane + 32 * i;
            if (e < E && pos[i] < 0) {
                const uint32_t key = order_key(a[i] + err[i]);
                if (key > bk) { bk = key; bs = i; }
            }
        }
        const uint32_t wk = __reduce_max_sync(0xffffffffu, bk);
        const uint32_t owners = __ballot_sync(0xffffffffu, wk != 0u && bk == wk);
        if (owners != 0u && lane == __ffs(owners) - 1) {
            probe_slot = bs;
            cand[n] = lane + 32 * bs;
        }
        __syncwarp();
        const int n_eval = n + (owners != 0u ? 1 : 0);
        exact_logits_all<T>(xrow, wg, bias, H, cand, n_eval, exact, lane);
    }

    // the error bound, checked wherever both values exist; a token that breaks it is evaluated over all experts
    bool nonfinite = n == 0;    // only NaN logits leave no candidate
    bool bad = false;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        if (pos[i] >= 0) bad |= !(fabsf(exact[pos[i]] - a[i]) <= err[i]);
        if (i == probe_slot) bad |= !(fabsf(exact[n] - a[i]) <= err[i]);
    }
    nonfinite = __any_sync(0xffffffffu, nonfinite);
    bad = __any_sync(0xffffffffu, bad);
    if (nonfinite || bad) {
        if (lane == 0 && dev_status) atomicOr(dev_status, nonfinite ? DEV_FAULT_NONFINITE : DEV_FAULT_SCREEN);
        __syncwarp();
        n = E;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) {
            const int e = lane + 32 * i;
            pos[i] = e < E ? e : -1;
            if (e < E) cand[e] = e;
        }
        __syncwarp();
        exact_logits_all<T>(xrow, wg, bias, H, cand, n, exact, lane);
    }
#pragma unroll
    for (int i = 0; i < SLOTS; ++i)
        if (pos[i] >= 0) {
            a[i] = exact[pos[i]];
            ekey[pos[i]] = order_key(a[i]);
        }
    __syncwarp();

    // top-k over the candidates' exact logits; the list ascends in expert index, so the lowest position among equal
    // values is the lowest index. Lane j keeps the j-th choice.
    int sel_e = 0;
    float sel_l = 0.0f;
#pragma unroll 1
    for (int j = 0; j < k; ++j) {
        uint32_t bk = 0u;
        int bc = 0x7fffffff;
        for (int c = lane; c < n; c += 32) {
            const uint32_t key = ekey[c];
            if (key > bk) { bk = key; bc = c; }
        }
        const uint32_t wk = __reduce_max_sync(0xffffffffu, bk);
        const int wc = min(__reduce_min_sync(0xffffffffu, bk == wk ? bc : 0x7fffffff), n - 1);
        if (lane == j) { sel_e = cand[wc]; sel_l = exact[wc]; }
        __syncwarp();
        if (lane == 0) ekey[wc] = 0u;
        __syncwarp();
    }

    float w;
    if (gate_fn == ARISTOS_GATE_SOFTMAX) {
        const float mx = __shfl_sync(0xffffffffu, sel_l, 0);
        float den = 0.0f;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i)
            if (lane + 32 * i < E) den += expf(a[i] - mx);
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) den += __shfl_xor_sync(0xffffffffu, den, m);
        w = expf(sel_l - mx) / den;
    } else {
        w = 1.0f / (1.0f + expf(-sel_l));
    }
    if (renorm) {
        float s = 0.0f;
        for (int j = 0; j < k; ++j) s += __shfl_sync(0xffffffffu, w, j);     // in choice order, like the other gate
        w = w / s;
    }
    if (lane < k) {
        topk_idx[(size_t)t * k + lane] = sel_e;
        topk_w[(size_t)t * k + lane] = w;
    }
}

bool screen_supported(int dtype, int H, int E, int k) {
    return (dtype == ARISTOS_DTYPE_BF16 || dtype == ARISTOS_DTYPE_F16) && E >= 32 && E <= GS_MAX_E && E % 4 == 0 &&
           H % 8 == 0 && k <= E && k <= MAX_TOPK;
}

template <typename T>
aristos_status_t launch_screened(const void* x, const void* wg, const float* bias, int S, int H, int E, int k,
                                 int gate_fn, int renorm, int32_t* topk_idx, float* topk_w, void* scratch,
                                 int32_t* dev_status, cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    float* wnorm = static_cast<float*>(scratch);
    float* partial = reinterpret_cast<float*>(static_cast<char*>(scratch) + GS_MAX_E * sizeof(float));
    GateScreenParams p;
    p.S = S; p.H = H; p.E = E;
    p.n_mma = ceil_div(E, 16) * 16;
    p.buf_cols = 32;
    while (p.buf_cols < p.n_mma) p.buf_cols *= 2;
    p.kblocks = ceil_div(H, GS_BK);
    p.slice_kb = GS_SLICE_KB > ceil_div(p.kblocks, GS_MAX_SLICES) ? GS_SLICE_KB : ceil_div(p.kblocks, GS_MAX_SLICES);
    p.nslices = ceil_div(p.kblocks, p.slice_kb);
    const int mtiles = ceil_div(S, GS_BM);
    int ysplit = device_sm_count() / mtiles;         // CTAs per token tile: fill the SMs, at most one per slice
    ysplit = ysplit < 1 ? 1 : (ysplit > p.nslices ? p.nslices : ysplit);
    p.bf16 = is_bf16 ? 1 : 0;
    p.partial = partial;
    p.dev_status = dev_status;

    CUtensorMap tmX, tmW;
    const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    ARISTOS_TRY(encode_map_3d(&tmX, dt, 2, x, H, S, 1, 128));
    ARISTOS_TRY(encode_map_3d(&tmW, dt, 2, wg, H, E, 1, 128));
    ARISTOS_CUDA_TRY(cudaFuncSetAttribute(gate_screen_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM_BYTES));

    gate_wnorm_kernel<T><<<ceil_div(E, 8), 256, 0, st>>>(static_cast<const T*>(wg), E, H, wnorm);
    ARISTOS_COUNT_LAUNCH();
    gate_screen_kernel<<<dim3(mtiles, ysplit), GS_THREADS, GS_SMEM_BYTES, st>>>(tmX, tmW, p);
    ARISTOS_COUNT_LAUNCH();
    // 4 n 2^-23 with n = the elements of H one slice accumulates
    const float err_scale = 4.0f * (float)(p.slice_kb * GS_BK) * 1.1920928955078125e-7f;
    const int sel_grid = ceil_div(S, SEL_WARPS);
#define ARISTOS_LAUNCH_SELECT(SLOTS)                                                                                 \
    gate_select_kernel<T, SLOTS><<<sel_grid, SEL_WARPS * 32, 0, st>>>(                                               \
        static_cast<const T*>(x), static_cast<const T*>(wg), bias, partial, p.nslices, wnorm, S, H, E, k, gate_fn,   \
        renorm, err_scale, topk_idx, topk_w, dev_status)
    if (E <= 64) ARISTOS_LAUNCH_SELECT(2);
    else if (E <= 128) ARISTOS_LAUNCH_SELECT(4);
    else ARISTOS_LAUNCH_SELECT(8);
#undef ARISTOS_LAUNCH_SELECT
    ARISTOS_COUNT_LAUNCH();
    ARISTOS_CUDA_TRY(cudaGetLastError());
    return ARISTOS_OK;
}

}  // namespace

}  // namespace aristos

using namespace aristos;

extern "C" size_t aristos_gate_scratch_bytes(int S, int E) {
    if (S <= 0 || E <= 0) return 0;
    const size_t bytes = GS_MAX_E * sizeof(float) + (size_t)GS_MAX_SLICES * S * E * sizeof(float);
    return (bytes + 255) / 256 * 256;
}

extern "C" aristos_status_t aristos_gate_topk_screened(const void* x, const void* w_gate, const float* gate_bias, int S,
                                                       int H, int E, int k, int gate_fn, int renorm, int dtype,
                                                       int32_t* topk_idx, float* topk_w, void* scratch,
                                                       size_t scratch_bytes, int32_t* dev_status, void* stream) {
    if (S < 0 || H <= 0 || E <= 0 || k <= 0) { set_last_error("gate: bad size"); return ARISTOS_ERR_INVALID_ARG; }
    // shapes the screen does not cover take the all-experts kernels: same routing either way
    if (!scratch || !screen_supported(dtype, H, E, k))
        return aristos_gate_topk(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, dtype, topk_idx, topk_w, nullptr,
                                 stream);
    if (!x || !w_gate || !topk_idx || !topk_w) { set_last_error("gate: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (!aligned16(x) || !aligned16(w_gate) || !aligned16(scratch)) {
        set_last_error("gate: pointers must be 16-byte aligned");
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (gate_fn != ARISTOS_GATE_SOFTMAX && gate_fn != ARISTOS_GATE_SIGMOID) return ARISTOS_ERR_INVALID_ARG;
    if (scratch_bytes < aristos_gate_scratch_bytes(S, E)) {
        set_last_error("gate: scratch of %zu bytes, %zu needed", scratch_bytes, aristos_gate_scratch_bytes(S, E));
        return ARISTOS_ERR_INVALID_ARG;
    }
    if (S == 0) return ARISTOS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == ARISTOS_DTYPE_BF16)
        return launch_screened<__nv_bfloat16>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w,
                                              scratch, dev_status, st);
    return launch_screened<__half>(x, w_gate, gate_bias, S, H, E, k, gate_fn, renorm, topk_idx, topk_w, scratch,
                                   dev_status, st);
}
