/*
 * aristos_moe.h - C ABI of the B200 (sm_100a) fused distributed MoE forward layer.
 *
 * The reference project (osayamenja/cuPlayground) exposes its MoE prototypes as zero-argument C++ harnesses that
 * allocate, launch and free inside one function (mma.cuh:371-443 testCollective, auditorium/combine.cuh:207-238
 * hostCombine, auditorium/overlap.cuh:159-242 overlapPrototype, auditorium/scheduling.cuh:267-288 and
 * warpScheduler.cuh:346-372 hostSchedule) and is configured by aristos_config.json (aristos_config.json:1-13,
 * aristos_config.schema.json:1-71, CMakeLists.txt:167-216). This header is the callable replacement of that
 * surface: the same configuration keys, the same tensor conventions (activations row-major (tokens, features),
 * weights row-major (out_features, in_features), fp32 accumulation - mma.cuh:394-397, :415-427), behind plain
 * pointers and sizes. No C++ or torch type crosses this boundary.
 *
 * Conventions
 *   - every tensor pointer is a DEVICE pointer, 16-byte aligned, unless the name ends in _host;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); calls are asynchronous
 *     with respect to it unless stated otherwise;
 *   - every function returns an aristos_status_t (never exits, never throws - the reference's CHECK_ERROR_EXIT,
 *     util.cuh:24-36, calls exit(1) instead);
 *   - there is no CPU fallback: without a usable CUDA device the compute entry points return ARISTOS_ERR_CUDA.
 */
#ifndef ARISTOS_MOE_H
#define ARISTOS_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ARISTOS_API __attribute__((visibility("default")))
#else
#define ARISTOS_API
#endif

typedef enum aristos_status {
    ARISTOS_OK = 0,
    ARISTOS_ERR_INVALID_ARG = 1,    /* NULL pointer, negative size, misaligned pointer */
    ARISTOS_ERR_CONFIG = 2,         /* configuration violates the schema or a kernel constraint */
    ARISTOS_ERR_IO = 3,             /* configuration file unreadable */
    ARISTOS_ERR_CUDA = 4,           /* a CUDA runtime/driver call failed (see aristos_last_error) */
    ARISTOS_ERR_NCCL = 5,           /* NCCL missing or a NCCL call failed */
    ARISTOS_ERR_UNSUPPORTED = 6,    /* valid request that this build does not implement */
    ARISTOS_ERR_WORKSPACE = 7,      /* caller-provided workspace too small */
    ARISTOS_ERR_DEVICE_TIMEOUT = 8, /* a bounded device-side wait expired (kernel returned early) */
    ARISTOS_ERR_DEVICE_BOUNDS = 9,  /* a routing-derived index was out of range (access skipped) */
    ARISTOS_ERR_NOMEM = 10,
    ARISTOS_ERR_GATE_SCREEN = 11,   /* the screened gate met an accumulation error above its bound: the affected token was
                                       re-evaluated exactly, but the bound cannot be trusted for these inputs
                                       (ARISTOS_GATE=exact selects the all-experts gate) */
    ARISTOS_ERR_NONFINITE = 12      /* a token's gate logits were NaN (non-finite activations or gate weights) */
} aristos_status_t;

/* torch_dtype (aristos_config.schema.json:54-58) and hidden_act (:24-28), with the extension values. */
enum { ARISTOS_DTYPE_F32 = 0, ARISTOS_DTYPE_TF32 = 1, ARISTOS_DTYPE_BF16 = 2, ARISTOS_DTYPE_F16 = 3,
       ARISTOS_DTYPE_FP8_E4M3 = 4 /* extension */ };
enum { ARISTOS_ACT_RELU = 0, ARISTOS_ACT_GELU = 1, ARISTOS_ACT_SWIGLU = 2 /* extension */,
       ARISTOS_ACT_IDENTITY = 3 /* extension, second projection */ };
enum { ARISTOS_GATE_SOFTMAX = 0, ARISTOS_GATE_SIGMOID = 1 };

/*
 * Layer description. The first eleven fields are the keys of aristos_config.json (aristos_config.json:2-12);
 * the reference turns them into -D macros at configure time (CMakeLists.txt:167-216), here they are read at run
 * time. The remaining fields are extension keys; a file that omits them gets the defaults shown.
 */
typedef struct aristos_config {
    double capacity_factor;   /* schema: integer >= 1; extension: any real >= 0 (1.25) */
    int drop_tokens;          /* 0: capacity = tokens (nothing is dropped); 1: capacity = ceil(cf*S*k/E) */
    int expert_top_k;
    int is_training;          /* read and ignored (forward only), as in the reference */
    int hidden_act;           /* ARISTOS_ACT_* */
    int hidden_size;          /* H, multiple of 64 */
    int intermediate_size;    /* I, multiple of 64 */
    int micro_batch;
    int num_experts;          /* E, global */
    int sequence_len;
    int torch_dtype;          /* ARISTOS_DTYPE_* */
    /* extension keys */
    int tokens;               /* "tokens": S per rank; 0 = micro_batch * sequence_len */
    int gate_fn;              /* "gate_fn": ARISTOS_GATE_*; default softmax */
    int renorm_topk;          /* "renorm_topk": divide the k weights by their sum; default 0 */
    double gate_bias_zipf_s;  /* "gate_bias_zipf_s": s > 0 adds -s*ln(e+1) to logit e; default 0 (off) */
    int ep_world;             /* "ep_world": ranks the experts are sharded over; default 1 */
    uint64_t seed;            /* "seed": only used by the synthetic-input helpers; default 0 */
} aristos_config_t;

/* Routing tensors of the last forward (device pointers owned by the layer handle, valid until destroy). */
typedef struct aristos_routing {
    const int32_t* topk_idx;       /* (S,k)   selected experts, by decreasing logit, ties -> lower index */
    const float* topk_w;           /* (S,k)   combine weights */
    const int32_t* count;          /* (E)     rows kept per expert (<= capacity) */
    const int32_t* slot_of;        /* (S,k)   expert*capacity + position, -1 = dropped */
    const int32_t* token_of_slot;  /* (E*cap) owning token of a slot, -1 = unused */
    int tokens, top_k, num_experts, capacity;
} aristos_routing_t;

typedef struct aristos_moe aristos_moe_t; /* opaque layer handle */

/* ---- status / errors ------------------------------------------------------------------------------------- */
ARISTOS_API const char* aristos_status_str(aristos_status_t s);
/* Text of the last failure on the calling thread (CUDA/NCCL error string, parser message). Never NULL. */
ARISTOS_API const char* aristos_last_error(void);
ARISTOS_API int aristos_version(void);

/* ---- configuration: replaces CMakeLists.txt:167-216 (JSON -> -D macros) ------------------------------------ */
ARISTOS_API aristos_status_t aristos_config_default(aristos_config_t* out); /* values of aristos_config.json:2-12 */
ARISTOS_API aristos_status_t aristos_config_parse(const char* json_text, aristos_config_t* out);
ARISTOS_API aristos_status_t aristos_config_load(const char* json_path, aristos_config_t* out);
/* Schema rules (aristos_config.schema.json) plus the kernel constraints of this build. */
ARISTOS_API aristos_status_t aristos_config_validate(const aristos_config_t* cfg);
ARISTOS_API int aristos_config_tokens(const aristos_config_t* cfg);   /* S per rank */
ARISTOS_API int aristos_config_capacity(const aristos_config_t* cfg); /* rows per expert per source rank */
/* Host helper: the Zipf prior of the skewed-routing case, bias_host[e] = -s*ln(e+1) as fp32. */
ARISTOS_API aristos_status_t aristos_zipf_bias_host(float* bias_host, int num_experts, double s);

/* ---- layer: replaces the allocate/launch/sync/free harnesses (mma.cuh:371-443, overlap.cuh:159-242) -------- */
/* nccl_unique_id: 128 bytes from aristos_nccl_unique_id on rank 0, shared by the caller; NULL when world == 1.
 * The CUDA device current at this call becomes the layer's device. */
ARISTOS_API aristos_status_t aristos_moe_create(const aristos_config_t* cfg, int rank, int world,
                                                const void* nccl_unique_id, aristos_moe_t** out);
ARISTOS_API aristos_status_t aristos_nccl_unique_id(void* out_128_bytes);
/* Host-only helpers that expose the layout logic of the expert-parallel exchange (no CUDA, no NCCL), so that it can
 * be checked with CPU ranks; they replace the symmetric-heap slot arithmetic of auditorium/overlap.cuh:28-35,183-190.
 * aristos_ep_exchange_plan writes up to max_entries rows {send_to, send_offset, recv_from, recv_offset, bytes} of the
 * exchange of one row window (the rank's own blocks first) and returns the number of transfers (-1 on bad arguments):
 * block (d*blocks_per_peer + b) of the send buffer goes to rank d and lands in block (src*blocks_per_peer + b) of
 * the receiver's buffer, `offset`/`len` select the window inside every block. aristos_ep_row_windows gives the row
 * windows a layer uses for a capacity. */
ARISTOS_API int aristos_ep_exchange_plan(int rank, int world, int blocks_per_peer, size_t block_stride, size_t offset,
                                         size_t len, int64_t* out, int max_entries);
ARISTOS_API aristos_status_t aristos_ep_row_windows(int cap, int* window_rows, int* windows);
ARISTOS_API size_t aristos_moe_workspace_bytes(const aristos_moe_t* layer);
/* Optional: hand the layer a caller-owned device workspace (>= aristos_moe_workspace_bytes, 1024-byte aligned).
 * Without it the first forward allocates one with cudaMalloc and keeps it until destroy. */
ARISTOS_API aristos_status_t aristos_moe_set_workspace(aristos_moe_t* layer, void* workspace, size_t bytes);
/* Optional expert biases used by every later forward (device pointers owned by the caller, NULL = none):
 * b1 (E_local, I), b3 (E_local, I; SwiGLU only), b2 (E_local, H), in the activations' dtype. */
ARISTOS_API aristos_status_t aristos_moe_set_bias(aristos_moe_t* layer, const void* b1, const void* b3,
                                                  const void* b2);
/*
 * One forward of the layer on this rank.
 *   x (S,H) activations          w_gate (E,H)        gate_bias (E) fp32 or NULL (NULL + gate_bias_zipf_s > 0 =
 *   the layer's own Zipf prior)   w1 (E_local,I,H)    w3 (E_local,I,H), SwiGLU only, else NULL
 *   w2 (E_local,H,I)             scales: fp8 only, else NULL          out (S,H), same dtype as x
 * torch_dtype 4 (fp8): x and out are bf16 (activations are quantised inside, per token and 128 elements); w1 / w3 /
 * w2 are e4m3; scales = fp32 [s1 (E_local, I/128, H/128) | s3 (same, SwiGLU only) | s2 (E_local, H/128, I/128)],
 * contiguous, as aristos_quantize_fp8(block_rows = 128) writes them. Across ranks the fp8 layer needs the "p2p"
 * transport (the gather stores quantised rows and scales straight into the owning rank's memory).
 * E_local = num_experts / world; rank r owns experts [r*E_local, (r+1)*E_local). Dropped tokens give zero rows.
 * Expert indices here are slots: which model expert a slot holds is the caller's choice (the rows of w_gate, the
 * entries of gate_bias and the expert weights follow it). A forward ends when the busiest rank's experts are done,
 * so a skewed routing prior wants its hot experts in slots of different ranks, e.g. expert e in slot
 * (e % world) * E_local + e / world (round-robin over the ranks).
 */
ARISTOS_API aristos_status_t aristos_moe_forward(aristos_moe_t* layer, const void* x, const void* w_gate,
                                                 const float* gate_bias, const void* w1, const void* w3,
                                                 const void* w2, const void* scales, void* out, void* stream);
/* Same call with HOST activations: copies x_host to the device, runs the forward, copies the result into
 * out_host and synchronises `stream` (the reference harness shape: host slab -> H2D -> kernels -> D2H,
 * mma.cuh:392-413, auditorium/overlap.cuh:192-237). Weights stay device-resident. */
ARISTOS_API aristos_status_t aristos_moe_forward_host(aristos_moe_t* layer, const void* x_host, const void* w_gate,
                                                      const float* gate_bias, const void* w1, const void* w3,
                                                      const void* w2, const void* scales, void* out_host,
                                                      void* stream);
/* The same, split in two so that consecutive calls overlap: aristos_moe_submit_host enqueues the host-to-device copy
 * (own copy stream), the forward (on `stream`) and the device-to-host copy (own copy stream) and returns; the copies
 * of one call run under the kernels of its neighbours. Four calls may be in flight (a fifth submit first waits for
 * the oldest); x_host / out_host must stay valid, and should be pinned, until aristos_moe_wait_host returns.
 * aristos_moe_forward_host == submit + wait. */
ARISTOS_API aristos_status_t aristos_moe_submit_host(aristos_moe_t* layer, const void* x_host, const void* w_gate,
                                                     const float* gate_bias, const void* w1, const void* w3,
                                                     const void* w2, const void* scales, void* out_host,
                                                     void* stream);
ARISTOS_API aristos_status_t aristos_moe_wait_host(aristos_moe_t* layer);
ARISTOS_API aristos_status_t aristos_moe_routing(const aristos_moe_t* layer, aristos_routing_t* out);
/* Copies the routing tensors of the last forward into host buffers sized as in aristos_routing_t (any pointer may
 * be NULL); synchronises the device first. */
ARISTOS_API aristos_status_t aristos_moe_routing_to_host(const aristos_moe_t* layer, int32_t* topk_idx_host,
                                                         float* topk_w_host, int32_t* count_host,
                                                         int32_t* slot_of_host, int32_t* token_of_slot_host);
/* Synchronises the layer's streams and reports device-side faults of the forwards since the last call
 * (ARISTOS_ERR_DEVICE_TIMEOUT / ARISTOS_ERR_DEVICE_BOUNDS / ARISTOS_ERR_GATE_SCREEN), then clears them.
 * Expert-parallel layers wait with a wall-clock limit (aristos_moe_set_timeout_ms): the reference's exchange spins
 * without bound on its peers' flags (auditorium/overlap.cuh:102-105, :133-136), so one stopped rank hangs all. Here,
 * when the last forward has not completed within the limit (a peer never sent its rows or its results), the rank
 * stores the current epoch into its own arrival flags from the host - every stream wait and kernel wait of that
 * forward then completes on whatever data is there -, marks the handle failed and returns
 * ARISTOS_ERR_DEVICE_TIMEOUT. A failed handle refuses further forwards (its epochs no longer match its peers');
 * aristos_moe_destroy still returns. aristos_moe_wait_host, aristos_moe_routing_to_host and aristos_moe_destroy
 * wait the same way. */
ARISTOS_API aristos_status_t aristos_moe_status(aristos_moe_t* layer);
/*
 * Training mode (is_training = 1; the reference's schema has the flag, aristos_config.schema.json:20-23, and nothing
 * behind it). Every forward of such a layer saves what a backward pass and the auxiliary load-balance loss need,
 * outside the working buffers that the next forward overwrites: the routing (topk_idx, topk_w, slot_of) and
 * load_balance = [frac (E) | prob (E) | aux | dropped]: frac[e] = share of the S*k assignments that chose expert e
 * (before drops), prob[e] = sum of the gate weights given to e / S, aux = E * sum frac*prob, dropped = share of
 * assignments that capacity dropped. By default the state lives in one layer-owned buffer (overwritten by the next
 * forward); aristos_moe_set_training_buffer points the NEXT forwards at a caller-owned device buffer of
 * aristos_moe_training_bytes() bytes (256-byte aligned; NULL = back to the layer's), so a caller keeps as many
 * micro-batches alive as it has buffers. aristos_moe_training_state returns the device pointers the LAST forward
 * wrote (valid in stream order after that forward). aristos_load_balance_stats is the stage on its own
 * (stats: aristos_load_balance_stats_bytes(E) bytes on the device).
 */
typedef struct aristos_training_state {
    const int32_t* topk_idx;      /* (tokens, top_k) */
    const float* topk_w;          /* (tokens, top_k) */
    const int32_t* slot_of;       /* (tokens, top_k), -1 = dropped */
    const float* load_balance;    /* 2 * num_experts + 2 floats */
    int tokens, top_k, num_experts;
} aristos_training_state_t;
ARISTOS_API size_t aristos_moe_training_bytes(const aristos_moe_t* layer);
ARISTOS_API aristos_status_t aristos_moe_set_training_buffer(aristos_moe_t* layer, void* device_buffer, size_t bytes);
ARISTOS_API aristos_status_t aristos_moe_training_state(const aristos_moe_t* layer, aristos_training_state_t* out);
/* Host copies of that state (any pointer may be NULL; load_balance_host: 2 * num_experts + 2 floats); synchronises. */
ARISTOS_API aristos_status_t aristos_moe_training_state_to_host(const aristos_moe_t* layer, int32_t* topk_idx_host,
                                                                float* topk_w_host, int32_t* slot_of_host,
                                                                float* load_balance_host);
ARISTOS_API size_t aristos_load_balance_stats_bytes(int E);
ARISTOS_API aristos_status_t aristos_load_balance_stats(const int32_t* topk_idx, const float* topk_w,
                                                        const int32_t* slot_of, int S, int k, int E, float* stats,
                                                        void* stream);
/* Wall-clock limit of those waits in milliseconds (default 30000, or ARISTOS_EP_TIMEOUT_MS at create). */
ARISTOS_API aristos_status_t aristos_moe_set_timeout_ms(aristos_moe_t* layer, int timeout_ms);
/* Stage stopwatch (the reference times its kernels with %globaltimer reads and cudaEvents, mma.cuh:56,163,
 * auditorium/overlap.cuh:207-224). With profiling on, every forward records CUDA events on its stream at the stage
 * boundaries; aristos_moe_stage_ms waits for the last forward and returns milliseconds, averaged over the forwards
 * since profiling was switched on (at most the last 64), for
 * {gate, dispatch + gather, expert FFN (with the exchanges when world > 1), combine, whole forward}. */
ARISTOS_API aristos_status_t aristos_moe_set_profiling(aristos_moe_t* layer, int enable);
ARISTOS_API aristos_status_t aristos_moe_stage_ms(aristos_moe_t* layer, float out_ms[5]);
/* Expert-parallel peer-memory layers (16-bit / tf32): milliseconds from the end of the dispatch bookkeeping until this
 * rank's count and gather kernels have stored its rows into the owning ranks and raised their flags (the part of the
 * "expert FFN" stage that is the outgoing exchange), averaged like aristos_moe_stage_ms; 0 for other layers. */
ARISTOS_API aristos_status_t aristos_moe_exchange_ms(aristos_moe_t* layer, float* sent_ms);
/* The same layers, the "expert FFN" stage split at its cross-rank waits (CUDA events on the caller's stream, averaged
 * like aristos_moe_stage_ms): out_ms = {dispatch end -> own rows sent (as aristos_moe_exchange_ms),
 * dispatch end -> every rank's row counts have arrived, counts arrived -> this rank's expert GEMMs (with the arrival
 * waits per source rank, the fused return stores and the return flags) are done, GEMMs done -> every rank's returned
 * rows have arrived}; zeros for other layers. The reference's overlap prototype times its exchange as a whole
 * (auditorium/overlap.cuh:206-236). */
ARISTOS_API aristos_status_t aristos_moe_exchange_profile(aristos_moe_t* layer, float out_ms[4]);
/* How the rows of an expert-parallel layer travel: "p2p" (the default: kernels store through the peers' CUDA-IPC
 * mapped exchange buffers over NVLink - the gather kernel writes every kept token row into the rank that owns its
 * expert, the down projection's epilogue writes every output tile into the rank the rows came from -, arrival is
 * published by epoch flags; the up projection waits per source rank inside the kernel, the combine behind a stream
 * memory wait. ARISTOS_EP_MODE=windows selects copy-engine pushes of padded row windows instead), "nccl" (grouped
 * ncclSend/ncclRecv; chosen with ARISTOS_EP_TRANSPORT=nccl, or by every rank together when any rank cannot allocate
 * or map the peer memory) or "none" (world == 1). */
ARISTOS_API const char* aristos_moe_ep_transport(const aristos_moe_t* layer);
/* Kernels launched by this library for `layer` since create (the benchmark's launch count). */
ARISTOS_API int64_t aristos_moe_launch_count(const aristos_moe_t* layer);
ARISTOS_API aristos_status_t aristos_moe_destroy(aristos_moe_t* layer);

/* ---- stage entry points (what the layer calls, exported for parity tests and for callers that fuse the
 *      stages into their own pipeline) ------------------------------------------------------------------------ */
/* Gate: logits = x * w_gate^T (+ gate_bias) in fp32 with a fixed reduction order, top-k on the logits (ties ->
 * lower expert index), softmax or sigmoid weights. The reference has no gate; its expert-tile contract
 * C = act(A*B^T + bias) with B stored (N,K) (mma.cuh:46-161) fixes the operand layout. logits_out may be NULL. */
ARISTOS_API aristos_status_t aristos_gate_topk(const void* x, const void* w_gate, const float* gate_bias, int S,
                                               int H, int E, int k, int gate_fn, int renorm, int dtype,
                                               int32_t* topk_idx, float* topk_w, float* logits_out, void* stream);
/* The same gate for many experts (what the layer calls when it needs no logits): a tcgen05 screen computes
 * approximate logits, the experts whose error interval reaches the k-th place are re-evaluated with the bit-exact
 * contract, top-k runs on those. topk_idx is identical to aristos_gate_topk's; softmax weights agree to rounding
 * (sigmoid weights exactly). Needs bf16/fp16 inputs and 32 <= E <= 256, E % 4 == 0; any other shape, or
 * scratch == NULL, runs aristos_gate_topk. scratch: aristos_gate_scratch_bytes(S, E) bytes, 16-byte aligned.
 * dev_status (device int32, may be NULL) receives fault bits of the bounded waits. */
ARISTOS_API size_t aristos_gate_scratch_bytes(int S, int E);
ARISTOS_API aristos_status_t aristos_gate_topk_screened(const void* x, const void* w_gate, const float* gate_bias,
                                                        int S, int H, int E, int k, int gate_fn, int renorm,
                                                        int dtype, int32_t* topk_idx, float* topk_w, void* scratch,
                                                        size_t scratch_bytes, int32_t* dev_status, void* stream);
/* Dispatch bookkeeping (capacity-bounded per-expert token lists, overflow dropped in token order). Replaces the
 * task-queue bookkeeping of auditorium/scheduling.cuh:218-252. scratch: aristos_dispatch_scratch_bytes(). */
ARISTOS_API size_t aristos_dispatch_scratch_bytes(int S, int k, int E);
ARISTOS_API aristos_status_t aristos_dispatch(const int32_t* topk_idx, int S, int k, int E, int cap,
                                              int32_t* count, int32_t* slot_of, int32_t* token_of_slot,
                                              void* scratch, size_t scratch_bytes, void* stream);
/*
 * Same dispatch, for callers that must not allocate device memory: a serving engine that has already handed all of
 * the GPU's memory to its own pool, or a latency-critical loop in which a cudaMalloc (which may synchronise the
 * device or simply fail) is not acceptable. It has no counterpart in the reference. The scratch is a fixed 64 KiB
 * array inside the library (held on every GPU that loads it until the process exits), so the sizes are limited to
 * S*k <= 131072 and E <= 256; larger requests are rejected with ARISTOS_ERR_CONFIG. The call allocates nothing.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
 * outside any stream capture. All calls share the one array and it keeps the previous call's contents: nothing in it
 * has to start at zero (the first kernel overwrites every entry the later ones read), but two calls whose kernels
 * overlap on the GPU (different streams, no ordering) race on it - order them.
 */
ARISTOS_API aristos_status_t aristos_dispatch_static(const int32_t* topk_idx, int S, int k, int E, int cap,
                                                     int32_t* count, int32_t* slot_of, int32_t* token_of_slot,
                                                     void* stream);
/* Gather token rows into expert-major order: xg[slot_of[t,j]] = x[t]. xg is (E*cap, H). */
ARISTOS_API aristos_status_t aristos_permute(const void* x, const int32_t* slot_of, int S, int k, int H, int dtype,
                                             void* xg, void* stream);
/*
 * Expert FFN over `groups` row groups of `rows_per_group` rows each; group g uses expert (g % experts) and has
 * count[g] valid rows. Only rows in [row_begin, row_end) of every group are computed (row_begin % 128 == 0; row_end a
 * multiple of 128 or equal to rows_per_group). Rows of y and h_scratch between count[g] and the end of the 128-row
 * tile that holds row count[g] - 1 may be overwritten with unspecified values; rows past that tile are not touched.
 *   h = act(xg * w1^T) or silu(xg * w1^T) * (xg * w3^T);   y = h * w2^T
 * Replaces fGET / deviceCollectiveMMA (mma.cuh:46-179, :198-369), BlockMM (processor/tiling.cuh:273-323) and the
 * in-kernel schedulers sK / wScheduler (auditorium/scheduling.cuh:202-265, warpScheduler.cuh:267-344).
 * h_scratch: (groups*rows_per_group, I) in dtype. dev_status: one int32 the kernels OR fault bits into (may be
 * NULL). sm_limit: CTAs of the persistent grid, 0 = all SMs.
 */
ARISTOS_API aristos_status_t aristos_expert_ffn(const void* xg, const int32_t* count, int groups,
                                                int rows_per_group, int experts, const void* w1, const void* w3,
                                                const void* w2, void* h_scratch, void* y, int H, int I,
                                                int hidden_act, int dtype, int row_begin, int row_end,
                                                int sm_limit, int32_t* dev_status, void* stream);
/* The same with the reference's bias operand: the epilogue is act(acc + bias) (FAA, processor/tiling.cuh:29-57; bias
 * tile (1,N), mma.cuh:87-95, :426-427). b1 (experts, I), b3 (experts, I; SwiGLU up projection), b2 (experts, H), in
 * the activations' dtype; any of them may be NULL. */
ARISTOS_API aristos_status_t aristos_expert_ffn_bias(const void* xg, const int32_t* count, int groups,
                                                     int rows_per_group, int experts, const void* w1, const void* w3,
                                                     const void* w2, const void* b1, const void* b3, const void* b2,
                                                     void* h_scratch, void* y, int H, int I, int hidden_act,
                                                     int dtype, int row_begin, int row_end, int sm_limit,
                                                     int32_t* dev_status, void* stream);
/*
 * FP8 (e4m3) operands with fp32 block scales (torch_dtype 4, extension; the reference lists fp8 e4m3 among its
 * tensor value types, util.cuh:70-76, but has no kernel for it).
 * aristos_quantize_fp8: src (mats, rows, cols) in bf16 or fp32 -> dst e4m3 and scales = amax / 448 per
 *   block_rows x 128 block: block_rows 1 = per row and 128 columns, scales (mats*rows, cols/128) - activations;
 *   block_rows 128 = per 128 x 128 block, scales (mats, ceil(rows/128), cols/128) - weights.
 * aristos_expert_ffn_fp8: like aristos_expert_ffn on quantised operands: xq (groups, rows, H) with sx
 *   (groups*rows, H/128); w1q / w3q (experts, I, H) with s1 / s3 (experts, I/128, H/128); w2q (experts, H, I) with
 *   s2 (experts, H/128, I/128). Every 128-wide K block is accumulated on the tensor cores and promoted with its
 *   scale in fp32. h is produced in bf16 (h_scratch), re-quantised per row and 128 columns (hq_scratch, sh_scratch)
 *   for the down projection; y is bf16. H and I must be multiples of 128.
 */
ARISTOS_API aristos_status_t aristos_quantize_fp8(const void* src, int64_t mats, int64_t rows, int cols,
                                                  int block_rows, int src_dtype, void* dst_fp8, float* scales,
                                                  void* stream);
ARISTOS_API aristos_status_t aristos_expert_ffn_fp8(const void* xq, const float* sx, const int32_t* count, int groups,
                                                    int rows_per_group, int experts, const void* w1q,
                                                    const float* s1, const void* w3q, const float* s3,
                                                    const void* w2q, const float* s2, void* h_scratch,
                                                    void* hq_scratch, float* sh_scratch, void* y, int H, int I,
                                                    int hidden_act, int row_begin, int row_end, int sm_limit,
                                                    int32_t* dev_status, void* stream);
/* Combine: out[t] = sum_j topk_w[t,j] * y[slot_of[t,j]] in increasing j (fp32), dropped assignments add
 * nothing. Replaces Combine / VAA / deviceCombine (auditorium/combine.cuh:19-205). */
ARISTOS_API aristos_status_t aristos_combine(const void* y, const int32_t* slot_of, const float* topk_w, int S,
                                             int k, int H, int dtype, void* out, void* stream);
/* Self-test of the failure path of the device-side waits (the reference's waits spin without bound:
 * auditorium/overlap.cuh:102-105, warpScheduler.cuh:339-341): one warp waits, with the routine the GEMM roles use, on a
 * barrier that nothing signals; the wait gives up after limit_ms, the kernel returns normally and the call reports
 * ARISTOS_ERR_DEVICE_TIMEOUT (that IS the expected result) with the time waited. The CUDA context stays usable. */
ARISTOS_API aristos_status_t aristos_selftest_bounded_wait(int limit_ms, int* waited_ms, void* stream);
/* The same for the wait on an arrival flag in global memory - what the up projection does before it loads the rows of
 * a source rank in the expert-parallel layer (the bounded successor of nvshmem_signal_wait_until,
 * auditorium/overlap.cuh:102-105): a flag word that nothing raises; ARISTOS_ERR_DEVICE_TIMEOUT is the expected
 * result. */
ARISTOS_API aristos_status_t aristos_selftest_bounded_flag_wait(int limit_ms, int* waited_ms, void* stream);
/* Tile shape of the tensor-core expert GEMM for later calls of this process (replaces the compile-time BLOCK_M /
 * BLOCK_N of processor/tiling.cuh:19-26): 0 automatic (CTA pairs, tcgen05 cta_group::2 with 256 x 256 tiles and groups
 * padded to whole tiles, where a row window holds >= 1024 rows; single-CTA 128 x 256 tiles otherwise), 1 single-CTA
 * tiles only, 2 pairs over each group's whole 256-row tiles + a single-CTA launch for its last < 256 rows, 3 padded
 * pairs for every window, -1 re-read ARISTOS_FFN_TILES (single | pair | pair-padded). Results are bit-identical
 * across the modes. */
ARISTOS_API aristos_status_t aristos_ffn_set_tile_mode(int mode);
/* Order in which the GEMM walks the row_tiles x col_tiles tiles of one row group (`band` row tiles per band; 0 = row
 * tile fastest): position `local` -> (row tile, column tile). Host-only, for tests. Returns 0, or -1 on bad input. */
ARISTOS_API int aristos_ffn_tile_coord(int local, int row_tiles, int col_tiles, int band, int* row_tile, int* col_tile);
/* Whether peer memory is the transport, given every rank's "works here" flag (all-gathered at create): only if it
 * works on all ranks; otherwise all ranks fall back together. Host-only, for tests of the agreement. */
ARISTOS_API int aristos_ep_transport_agreed(const int* ok_flags, int world);
/* The arrival-flag protocol of the peer-memory transport on plain host words, as the kernels and stream waits apply it
 * to a rank's flag page (successor of the reference's signal values, auditorium/overlap.cuh:20-24, :100-105): a page
 * of aristos_ep_flag_words() 32-bit words; word aristos_ep_flag_word_index(kind, window, src) (kind 0 rows in, 1
 * results back, 2 counts) holds the last epoch rank src published; aristos_ep_flags_pending returns the set of source
 * ranks (bit s) whose flag has not reached `epoch` (cyclic comparison); aristos_ep_flags_release is what a rank does
 * to its OWN page when its time limit expires: every lagging word takes the epoch, nothing stays pending. Host-only;
 * the tests run the protocol among CPU ranks with them. */
ARISTOS_API int aristos_ep_flag_words(void);
ARISTOS_API int aristos_ep_flag_word_index(int kind, int window, int src);
ARISTOS_API uint32_t aristos_ep_flags_pending(const uint32_t* words, uint32_t epoch, int world, int kind, int window);
ARISTOS_API void aristos_ep_flags_release(uint32_t* words, uint32_t epoch);
/* The order in which the expert GEMMs walk `groups` row groups of `experts` experts (group g uses expert
 * g % experts): position -> group, a permutation that keeps the groups of one expert adjacent. Host-only, for tests. */
ARISTOS_API int aristos_ffn_group_order(int position, int groups, int experts);
/* The same order on a rank of an expert-parallel layer: inside an expert the source ranks are taken in ring order
 * starting at first_source (the rank itself: its own rows are in its memory before the kernel starts). */
ARISTOS_API int aristos_ffn_group_order_from(int position, int groups, int experts, int first_source);
/* Dense packing of the rows an expert receives from all source ranks (the fp8 expert-parallel layer), host-side run of
 * what the layer computes on the device from the all-gathered counts allcount[src * E + e]: send_base[e] (E entries) =
 * first row of THIS rank's rows inside expert e's group at its owner (the lower ranks' rows come first); for the
 * experts this rank owns, dense_count[el] (E_local entries) = rows received in all and src_off[el * (world + 1) + s] =
 * first row of source s (entry `world` = the total). Host-only, for tests. */
ARISTOS_API aristos_status_t aristos_ep_dense_plan_host(const int32_t* allcount, int world, int E, int E_local, int rank,
                                                        int32_t* send_base, int32_t* dense_count, int32_t* src_off);
/* Synthetic inputs: Philox4x32-10 + Box-Muller normal fill (the reference draws inputs from Philox,
 * main.cu:22-31). Element i uses counter (i/4, 0, stream_id, 0), key = seed, output word i%4. */
ARISTOS_API aristos_status_t aristos_fill_normal(void* dst, int64_t n, float mean, float std, uint64_t seed,
                                                 uint32_t stream_id, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ARISTOS_MOE_H */
