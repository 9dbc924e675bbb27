/*
 * CPU oracle for the fused MoE forward path (gate -> dispatch -> expert FFN -> combine).
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library links, loads or calls this file; it is the checker
 * for the CUDA path and the timed CPU baseline of the benchmark.
 *
 * PARITY STATUS: "parity unpinned" for the MoE semantics. The reference tree (osayamenja/cuPlayground) holds no
 * gate, no dispatch, no capacity logic, no CPU path and no test or golden vector for them, and its GPU harnesses
 * cannot be built offline (they include cuBLASDx / CUTLASS@main / NVSHMEM, none of which is vendored). What the
 * reference does pin, and what this file follows:
 *   - expert tile contract  C = act(A * B^T + bias), A (M,K) row-major, B (N,K) row-major ("weights are
 *     (out_features, in_features)"), fp32 accumulation, conversion on store        mma.cuh:46-161, :394-397, :415-427
 *   - epilogue = activation(accumulator + term)                                   processor/tiling.cuh:29-57
 *   - combine accumulates expert rows into the token's own row, float being the
 *     "safe accumulator type"                                                     auditorium/combine.cuh:19-34, :170-186
 *   - config keys and enums (hidden_act 0 relu / 1 gelu, torch_dtype 0..3)        aristos_config.schema.json:6-58
 * The hand-written fixtures of the reference harnesses give known answers that tests/ replay against this file:
 *   mma.cuh:399-411 (2x2 corner GEMM + bias + ReLU), benchmarks.cuh:480-488 (broadcast bias),
 *   auditorium/combine.cuh:219-231 (identity-index combine).
 *
 * Semantics the reference leaves open and this oracle fixes (they are the specification of the CUDA path):
 *   - gate logit reduction order (bit-exact contract, see orc_gate_logits)
 *   - top-k on logits, ties -> lower expert index
 *   - capacity = ceil(cf * S * k / E) when drop_tokens, else S; position of (t,j) in expert e = number of
 *     assignments to e that come earlier in token-major order; kept iff position < capacity
 *   - combine weights are computed before drops; a dropped assignment contributes zero
 *   - GELU is the exact erf form (what cutlass::epilogue::thread::GELU computes)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------------------------------------------------------
 * Philox4x32-10 + Box-Muller input generator (the reference draws its inputs from Philox too: main.cu:22-31).
 * Element i of a tensor uses counter (i/4, 0, stream, 0), key (seed_lo, seed_hi) and output word i%4.
 * ------------------------------------------------------------------------------------------------------------- */
static inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

ORC_API void orc_fill_normal(float* out, int64_t n, float mean, float std, uint64_t seed, uint32_t stream) {
    const int64_t nblk = (n + 3) / 4;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblk; ++b) {
        uint32_t c[4] = {(uint32_t)b, (uint32_t)((uint64_t)b >> 32), stream, 0u};
        philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
        float z[4];
        for (int h = 0; h < 2; ++h) {
            /* u1 in (0,1], u2 in [0,1) */
            float u1 = ((float)(c[2 * h] >> 8) + 1.0f) * (1.0f / 16777216.0f);
            float u2 = (float)(c[2 * h + 1] >> 8) * (1.0f / 16777216.0f);
            float r = sqrtf(-2.0f * logf(u1));
            float th = 6.283185307179586f * u2;
            z[2 * h] = r * cosf(th);
            z[2 * h + 1] = r * sinf(th);
        }
        for (int j = 0; j < 4; ++j) {
            int64_t i = 4 * b + j;
            if (i < n) out[i] = mean + std * z[j];
        }
    }
}

/* Round fp32 values to the nearest bf16 (ties to even) and keep them as fp32. */
ORC_API void orc_round_bf16(float* v, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u; memcpy(&u, &v[i], 4);
        if ((u & 0x7F800000u) != 0x7F800000u) {
            u += 0x7FFFu + ((u >> 16) & 1u);
        }
        u &= 0xFFFF0000u;
        memcpy(&v[i], &u, 4);
    }
}

/* ---------------------------------------------------------------------------------------------------------------
 * Capacity. cap = ceil(cf*S*k/E) when tokens are dropped on overflow, else S (an expert can receive a token at
 * most once, so S rows always suffice). The fp32 reference case (S=128, E=8, k=1, cf=1) gives cap = S/E = 16.
 * ------------------------------------------------------------------------------------------------------------- */
ORC_API int orc_capacity(int S, int E, int k, double cf, int drop_tokens) {
    if (!drop_tokens) return S;
    double c = ceil(cf * (double)S * (double)k / (double)E - 1e-9);
    if (c < 1.0) c = 1.0;
    if (c > (double)S) c = (double)S;
    return (int)c;
}

/* Zipf prior added to the gate logits of the skewed-routing stress case: bias_e = -s * ln(e + 1). */
ORC_API void orc_zipf_bias(float* bias, int E, double s) {
    for (int e = 0; e < E; ++e) bias[e] = (float)(-s * log((double)(e + 1)));
}

/* ---------------------------------------------------------------------------------------------------------------
 * Gate logits, bit-exact contract.
 *   logit[t,e] = tree( P[0..31] ) (+ bias[e]),   P[c] = p[c][0] + p[c][1],
 *   p[c][h % 2] accumulates, in increasing h, fmaf(x[t,h], wg[e,h], p[c][h % 2]) over the 8-element chunks
 *   q = h/8 with q % 32 == c (even and odd elements separately); the tree is the xor butterfly 16, 8, 4, 2, 1
 *   (P[c] = P[c] + P[c ^ m]).
 * This is the order a warp produces when lane c owns every 32nd 16-byte chunk of a bf16 row and multiplies the
 * (even, odd) element pairs with packed two-lane fused multiply-adds.
 * x is (S,H) row-major, wg is (E,H) row-major (the reference's B-operand convention, mma.cuh:396-397).
 * ------------------------------------------------------------------------------------------------------------- */
static float gate_logit_one(const float* xr, const float* wr, int H) {
    float pe[32], po[32], p[32];
    for (int c = 0; c < 32; ++c) pe[c] = po[c] = 0.0f;
    const int nchunk = H / 8;
    for (int q = 0; q < nchunk; ++q) {
        const int c = q & 31;
        float ae = pe[c], ao = po[c];
        for (int v = 0; v < 8; v += 2) {
            ae = fmaf(xr[q * 8 + v], wr[q * 8 + v], ae);
            ao = fmaf(xr[q * 8 + v + 1], wr[q * 8 + v + 1], ao);
        }
        pe[c] = ae; po[c] = ao;
    }
    for (int c = 0; c < 32; ++c) p[c] = pe[c] + po[c];
    for (int m = 16; m >= 1; m >>= 1) {
        float np[32];
        for (int c = 0; c < 32; ++c) np[c] = p[c] + p[c ^ m];
        for (int c = 0; c < 32; ++c) p[c] = np[c];
    }
    return p[0];
}

ORC_API void orc_gate_logits(const float* x, const float* wg, const float* bias, int S, int H, int E,
                             float* logits) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < S; ++t)
        for (int e = 0; e < E; ++e) {
            float l = gate_logit_one(x + (size_t)t * H, wg + (size_t)e * H, H);
            if (bias) l = l + bias[e];
            logits[(size_t)t * E + e] = l;
        }
}

/* Top-k over logits (strict '>' scan from e = 0, so ties go to the lower index), then the combine weights:
 * gate_fn 0: softmax over all E experts; gate_fn 1: sigmoid. renorm: divide by the sum of the k selected. */
ORC_API void orc_gate_topk(const float* logits, int S, int E, int k, int gate_fn, int renorm,
                           int32_t* topk_idx, float* topk_w) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < S; ++t) {
        const float* l = logits + (size_t)t * E;
        int32_t* idx = topk_idx + (size_t)t * k;
        float* w = topk_w + (size_t)t * k;
        for (int j = 0; j < k; ++j) {
            int best = -1;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int i = 0; i < j; ++i) taken |= (idx[i] == e);
                if (taken) continue;
                if (best < 0 || l[e] > l[best]) best = e;
            }
            idx[j] = best;
        }
        if (gate_fn == 0) {
            float mx = l[idx[0]];
            double den = 0.0;
            for (int e = 0; e < E; ++e) den += exp((double)(l[e] - mx));
            for (int j = 0; j < k; ++j) w[j] = (float)(exp((double)(l[idx[j]] - mx)) / den);
        } else {
            for (int j = 0; j < k; ++j) w[j] = (float)(1.0 / (1.0 + exp(-(double)l[idx[j]])));
        }
        if (renorm) {
            double s = 0.0;
            for (int j = 0; j < k; ++j) s += (double)w[j];
            for (int j = 0; j < k; ++j) w[j] = (float)((double)w[j] / s);
        }
    }
}

/* ---------------------------------------------------------------------------------------------------------------
 * Dispatch: serial walk in token-major order, so "overflow dropped in token order" holds by construction.
 *   count[e]            rows kept for expert e (<= cap)
 *   slot_of[t*k+j]      e*cap + position, or -1 when the assignment was dropped
 *   token_of_slot[s]    token that owns slot s, or -1 for an unused slot (E*cap entries)
 * ------------------------------------------------------------------------------------------------------------- */
ORC_API void orc_dispatch(const int32_t* topk_idx, int S, int k, int E, int cap,
                          int32_t* count, int32_t* slot_of, int32_t* token_of_slot) {
    for (int e = 0; e < E; ++e) count[e] = 0;
    for (int64_t s = 0; s < (int64_t)E * cap; ++s) token_of_slot[s] = -1;
    for (int t = 0; t < S; ++t)
        for (int j = 0; j < k; ++j) {
            const int e = topk_idx[(size_t)t * k + j];
            if (count[e] < cap) {
                const int s = e * cap + count[e];
                slot_of[(size_t)t * k + j] = s;
                token_of_slot[s] = t;
                count[e] += 1;
            } else {
                slot_of[(size_t)t * k + j] = -1;
            }
        }
}

/* ---------------------------------------------------------------------------------------------------------------
 * Expert tile: C = act(A * B^T + bias)   (mma.cuh:46-161; processor/tiling.cuh:29-57)
 * A (M,K) row-major, B (N,K) row-major, C (M,N) row-major, bias (N) or NULL, fp32 accumulation.
 * act: 0 relu, 1 gelu (erf), 3 identity.
 * ------------------------------------------------------------------------------------------------------------- */
static inline float act_apply(float v, int act) {
    switch (act) {
        case 0: return v > 0.0f ? v : 0.0f;
        case 1: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
        default: return v;
    }
}
static inline float silu(float v) { return v / (1.0f + expf(-v)); }

static inline float round_bf16_one(float v) {
    uint32_t u; memcpy(&u, &v, 4);
    if ((u & 0x7F800000u) != 0x7F800000u) u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    memcpy(&v, &u, 4);
    return v;
}

/* Nearest fp8 e4m3 value (ties to even, saturating at +-448), returned as fp32. */
static inline float e4m3_round(float f) {
    float a = fabsf(f);
    if (!(a < 448.0f)) a = 448.0f;
    else if (a < 0.015625f) a = rintf(a * 512.0f) * (1.0f / 512.0f);             /* subnormals: step 2^-9 */
    else {
        int ex;
        frexpf(a, &ex);                                                          /* a = m * 2^ex, m in [0.5, 1) */
        const float step = ldexpf(1.0f, ex - 4);                                 /* 2^(E-3), E = ex - 1 */
        a = rintf(a / step) * step;
        if (a > 448.0f) a = 448.0f;
    }
    return copysignf(a, f);
}

/* What an fp8 pipeline stores for a row of hidden activations: bf16 rounding, then e4m3 with one scale
 * (amax / 448) per 128 consecutive values; returned de-quantised. */
static void quantize_row_fp8_inplace(float* h, int n) {
    for (int i = 0; i < n; ++i) h[i] = round_bf16_one(h[i]);
    for (int g0 = 0; g0 < n; g0 += 128) {
        const int len = n - g0 < 128 ? n - g0 : 128;
        float amax = 0.0f;
        for (int i = 0; i < len; ++i) { const float a = fabsf(h[g0 + i]); if (a > amax) amax = a; }
        const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
        const float inv = 1.0f / scale;
        for (int i = 0; i < len; ++i) h[g0 + i] = e4m3_round(h[g0 + i] * inv) * scale;
    }
}

static inline float dotf(const float* a, const float* b, int K) {
    /* 16 independent partial sums so the compiler can vectorise without reassociation flags */
    float p[16];
    for (int i = 0; i < 16; ++i) p[i] = 0.0f;
    int k = 0;
    for (; k + 16 <= K; k += 16)
        for (int i = 0; i < 16; ++i) p[i] += a[k + i] * b[k + i];
    float s = 0.0f;
    for (; k < K; ++k) s += a[k] * b[k];
    for (int i = 0; i < 16; ++i) s += p[i];
    return s;
}

ORC_API void orc_gemm_bias_act(const float* A, const float* B, const float* bias, float* C,
                               int M, int N, int K, int act) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float v = dotf(A + (size_t)m * K, B + (size_t)n * K, K);
            if (bias) v += bias[n];
            C[(size_t)m * N + n] = act_apply(v, act);
        }
}

/* Expert FFN over the gathered rows of every expert.
 *   xg (E, cap, H); w1 (E, I, H); w3 (E, I, H) or NULL; w2 (E, H, I); y (E, cap, H)
 *   optional biases b1 (E, I), b3 (E, I), b2 (E, H): every projection is act(acc + bias) (processor/tiling.cuh:29-57)
 *   hidden_act 0 relu, 1 gelu: h = act(xg w1^T); 2 swiglu: h = silu(xg w1^T) * (xg w3^T);  y = h w2^T
 * Rows at or past count[e] are left untouched. round_h 1 rounds h to bf16 (what a bf16 pipeline stores), 2 rounds it
 * to bf16 and then to e4m3 with one scale per 128 values (what the fp8 pipeline feeds its down projection). */
ORC_API void orc_expert_ffn(const float* xg, const int32_t* count, const float* w1, const float* w3,
                            const float* w2, const float* b1, const float* b3, const float* b2, float* y, int E,
                            int cap, int H, int I, int hidden_act, int round_h) {
    int64_t total = 0;
    for (int e = 0; e < E; ++e) total += count[e];
    int32_t* row_e = (int32_t*)malloc(sizeof(int32_t) * (size_t)(total > 0 ? total : 1));
    int32_t* row_r = (int32_t*)malloc(sizeof(int32_t) * (size_t)(total > 0 ? total : 1));
    int64_t n = 0;
    for (int e = 0; e < E; ++e)
        for (int r = 0; r < count[e]; ++r) { row_e[n] = e; row_r[n] = r; ++n; }
#pragma omp parallel
    {
        float* h = (float*)malloc(sizeof(float) * (size_t)I);
#pragma omp for schedule(dynamic, 4)
        for (int64_t i = 0; i < total; ++i) {
            const int e = row_e[i];
            const size_t row = (size_t)e * cap + row_r[i];
            const float* xr = xg + row * H;
            const float* W1 = w1 + (size_t)e * I * H;
            const float* W3 = w3 ? w3 + (size_t)e * I * H : NULL;
            const float* W2 = w2 + (size_t)e * H * I;
            for (int n1 = 0; n1 < I; ++n1) {
                float g = dotf(xr, W1 + (size_t)n1 * H, H);
                if (b1) g += b1[(size_t)e * I + n1];
                float v;
                if (hidden_act == 2) {
                    float u = dotf(xr, W3 + (size_t)n1 * H, H);
                    if (b3) u += b3[(size_t)e * I + n1];
                    v = silu(g) * u;
                } else {
                    v = act_apply(g, hidden_act);
                }
                h[n1] = v;
            }
            if (round_h == 1) {
                for (int n1 = 0; n1 < I; ++n1) h[n1] = round_bf16_one(h[n1]);
            } else if (round_h == 2) {
                quantize_row_fp8_inplace(h, I);
            }
            float* yr = y + row * H;
            for (int n2 = 0; n2 < H; ++n2) {
                float v = dotf(h, W2 + (size_t)n2 * I, I);
                if (b2) v += b2[(size_t)e * H + n2];
                yr[n2] = v;
            }
        }
        free(h);
    }
    free(row_e); free(row_r);
}

/* Gather: xg[slot] = x[token_of_slot[slot]] for used slots (unused rows are zeroed). */
ORC_API void orc_permute(const float* x, const int32_t* token_of_slot, int64_t nslots, int H, float* xg) {
#pragma omp parallel for schedule(static)
    for (int64_t s = 0; s < nslots; ++s) {
        const int t = token_of_slot[s];
        if (t >= 0) memcpy(xg + (size_t)s * H, x + (size_t)t * H, sizeof(float) * (size_t)H);
        else memset(xg + (size_t)s * H, 0, sizeof(float) * (size_t)H);
    }
}

/* Combine: out[t] = sum_j w[t,j] * y[slot_of[t,j]] in increasing j, fp32 accumulation
 * (auditorium/combine.cuh:19-34: float is the accumulator type); dropped assignments add nothing. */
ORC_API void orc_combine(const float* y, const int32_t* slot_of, const float* topk_w, int S, int k, int H,
                         float* out) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < S; ++t) {
        float* o = out + (size_t)t * H;
        for (int h = 0; h < H; ++h) o[h] = 0.0f;
        for (int j = 0; j < k; ++j) {
            const int s = slot_of[(size_t)t * k + j];
            if (s < 0) continue;
            const float w = topk_w[(size_t)t * k + j];
            const float* yr = y + (size_t)s * H;
            for (int h = 0; h < H; ++h) o[h] = fmaf(w, yr[h], o[h]);
        }
    }
}

/* ---------------------------------------------------------------------------------------------------------------
 * Whole layer on one rank. All tensors fp32 on the host (already rounded to the storage type of the GPU run).
 * Optional outputs (may be NULL): topk_idx, topk_w (S*k), count (E), slot_of (S*k), token_of_slot (E*cap).
 * Token rows are computed directly from the routing (no (E,cap,H) staging buffers), so the full-size configs fit.
 * only_rows: if n_only > 0, only those tokens' output rows are computed (sampled parity at full size).
 * x_ffn: if not NULL, the experts read these activations (e.g. de-quantised fp8) while the gate reads x.
 * ------------------------------------------------------------------------------------------------------------- */
ORC_API int orc_moe_forward(const float* x, const float* wg, const float* gate_bias, const float* w1,
                            const float* w3, const float* w2, int S, int H, int I, int E, int k, int cap,
                            int gate_fn, int renorm, int hidden_act, int round_h, float* out,
                            int32_t* topk_idx_o, float* topk_w_o, int32_t* count_o, int32_t* slot_of_o,
                            int32_t* token_of_slot_o, const int32_t* only_rows, int n_only, const float* x_ffn) {
    float* logits = (float*)malloc(sizeof(float) * (size_t)S * E);
    int32_t* idx = (int32_t*)malloc(sizeof(int32_t) * (size_t)S * k);
    float* tw = (float*)malloc(sizeof(float) * (size_t)S * k);
    int32_t* count = (int32_t*)malloc(sizeof(int32_t) * (size_t)E);
    int32_t* slot_of = (int32_t*)malloc(sizeof(int32_t) * (size_t)S * k);
    int32_t* tos = (int32_t*)malloc(sizeof(int32_t) * (size_t)E * cap);
    if (!logits || !idx || !tw || !count || !slot_of || !tos) return 1;
    orc_gate_logits(x, wg, gate_bias, S, H, E, logits);
    orc_gate_topk(logits, S, E, k, gate_fn, renorm, idx, tw);
    orc_dispatch(idx, S, k, E, cap, count, slot_of, tos);

    const int nrows = n_only > 0 ? n_only : S;
    if (out) {
#pragma omp parallel
        {
            float* h = (float*)malloc(sizeof(float) * (size_t)I);
#pragma omp for schedule(dynamic, 2)
            for (int r = 0; r < nrows; ++r) {
                const int t = n_only > 0 ? only_rows[r] : r;
                float* o = out + (size_t)r * H;
                for (int c = 0; c < H; ++c) o[c] = 0.0f;
                const float* xr = (x_ffn ? x_ffn : x) + (size_t)t * H;   /* experts may see quantised activations */
                for (int j = 0; j < k; ++j) {
                    if (slot_of[(size_t)t * k + j] < 0) continue;
                    const int e = idx[(size_t)t * k + j];
                    const float w = tw[(size_t)t * k + j];
                    const float* W1 = w1 + (size_t)e * I * H;
                    const float* W3 = w3 ? w3 + (size_t)e * I * H : NULL;
                    const float* W2 = w2 + (size_t)e * H * I;
                    for (int n1 = 0; n1 < I; ++n1) {
                        float g = dotf(xr, W1 + (size_t)n1 * H, H);
                        float v;
                        if (hidden_act == 2) v = silu(g) * dotf(xr, W3 + (size_t)n1 * H, H);
                        else v = act_apply(g, hidden_act);
                        if (round_h == 1) v = round_bf16_one(v);
                        h[n1] = v;
                    }
                    if (round_h == 2) quantize_row_fp8_inplace(h, I);
                    for (int n2 = 0; n2 < H; ++n2) o[n2] = fmaf(w, dotf(h, W2 + (size_t)n2 * I, I), o[n2]);
                }
            }
            free(h);
        }
    }
    if (topk_idx_o) memcpy(topk_idx_o, idx, sizeof(int32_t) * (size_t)S * k);
    if (topk_w_o) memcpy(topk_w_o, tw, sizeof(float) * (size_t)S * k);
    if (count_o) memcpy(count_o, count, sizeof(int32_t) * (size_t)E);
    if (slot_of_o) memcpy(slot_of_o, slot_of, sizeof(int32_t) * (size_t)S * k);
    if (token_of_slot_o) memcpy(token_of_slot_o, tos, sizeof(int32_t) * (size_t)E * cap);
    free(logits); free(idx); free(tw); free(count); free(slot_of); free(tos);
    return 0;
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Number of OpenMP threads for the later calls of this process. A launcher may have exported OMP_NUM_THREADS=1
 * (torch.distributed.run does); the benchmark's CPU arm sets the count from the cores it may use instead. */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
