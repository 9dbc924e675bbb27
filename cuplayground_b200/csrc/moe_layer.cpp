// Layer handle: workspace planning and the orchestration gate -> dispatch -> (all-to-all) -> expert FFN ->
// (all-to-all) -> combine behind aristos_moe_forward.
//
// Replaces the reference's host harnesses, which allocate one slab, copy inputs in, launch and synchronise inside a
// zero-argument function (mma.cuh:371-443 testCollective; auditorium/overlap.cuh:159-242 overlapPrototype, whose
// per-peer pipeline "put tile -> wait flag -> GEMM -> put result -> wait flag" (:94-153) becomes the chunked
// exchange below: rows travel in row windows of every expert block, the GEMMs of window c run while window c+1 is
// still in flight, and the results of window c return while window c+1 is being computed).
#include <nvtx3/nvToolsExt.h>

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <thread>
#include <vector>

#include "common.cuh"
#include "ep_nccl.h"
#include "ep_p2p.h"
#include "ep_kernels.h"
#include "ffn_internal.h"

namespace aristos {
aristos_status_t dispatch_impl(const int32_t* topk_idx, int S, int k, int E, int cap, int32_t* count,
                               int32_t* slot_of, int32_t* token_of_slot, void* scratch, size_t scratch_bytes,
                               int32_t* dev_status, cudaStream_t st);
}

using namespace aristos;

struct aristos_moe {
    aristos_config_t cfg;
    int rank = 0, world = 1, device = 0;
    int S = 0, H = 0, I = 0, E = 0, k = 0, cap = 0, E_local = 0, groups = 0;
    size_t elt = 2;
    // workspace
    void* ws = nullptr;
    size_t ws_bytes = 0;
    bool ws_owned = false;
    // carve-up of the workspace
    int32_t *topk_idx = nullptr, *count = nullptr, *slot_of = nullptr, *token_of_slot = nullptr, *rcount = nullptr,
            *dev_status = nullptr;
    float *topk_w = nullptr, *gate_bias = nullptr;
    // fp8 path (torch_dtype 4): quantised activations, their scales, and the re-quantised hidden activations
    bool fp8 = false;
    void *xq = nullptr, *xgq = nullptr, *hq = nullptr;
    float *sx = nullptr, *sxg = nullptr, *sh = nullptr;
    void *dispatch_scratch = nullptr, *xg = nullptr, *xr = nullptr, *h = nullptr, *yr = nullptr, *yg = nullptr;
    // host-activation path: staging slots, so that the copy-in of one call, the kernels of another and the copy-out
    // of a third run at once (a forward shorter than its copies needs three in flight to keep both copy engines busy)
    static constexpr int HOST_SLOTS = 4;
    struct HostSlot {
        void *x_dev = nullptr, *out_dev = nullptr;
        cudaEvent_t h2d_done = nullptr, compute_done = nullptr, d2h_done = nullptr;
        bool busy = false;
    } slots[HOST_SLOTS];
    int slot_next = 0;
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    size_t dispatch_scratch_bytes = 0;
    void* gate_scratch = nullptr;            // screened gate: expert norms and split partial logits
    size_t gate_scratch_bytes = 0;
    bool bias_ready = false;
    // expert parallel
    EpComm* comm = nullptr;
    EpP2P* p2p = nullptr;                    // peer-memory transport (rows pushed by the copy engines); else NCCL
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_dispatched = nullptr, ev_returned = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_out;
    int chunks = 1, chunk_rows = 0, ffn_sm_limit = 0;
    bool ep_direct = false;                  // p2p: gather/return kernels store through peer pointers
    int direct_windows = 1;                  // row windows of the direct mode (gather / GEMMs / return pipelined)
    bool fused_return = false;               // direct mode: the down projection's epilogue stores into the source ranks
    bool kernel_wait = false;                // direct mode: the up projection waits for each source's rows itself
    bool overlap_gather = false;             // direct mode: rows for other ranks are gathered beside the up projection
    bool dense = false;                      // fp8 across ranks: received rows packed per expert across the sources
    int32_t *send_base = nullptr, *dense_count = nullptr, *src_off = nullptr;
    int32_t* ffn_done = nullptr;             // counters of the one-launch expert FFN (groups x row tiles)
    size_t ffn_done_ints = 0;
    int64_t launches = 0;
    const void *b1 = nullptr, *b3 = nullptr, *b2 = nullptr;   // optional expert biases (caller-owned, device)
    // failure handling of the exchange: every wait for a forward's completion has a wall-clock limit; on expiry the
    // rank releases its own flag waits, and the handle refuses further forwards (its epochs no longer match the peers')
    int timeout_ms = 30000;
    bool failed = false;
    cudaEvent_t ev_last = nullptr;           // end of the last forward on its stream
    bool ev_last_valid = false;
    // training mode (is_training = 1): routing of the last forward kept for a backward pass + load-balance statistics
    void* train_own = nullptr;               // layer-owned buffer (in the workspace)
    void* train_buf = nullptr;               // where the next forward saves: caller's buffer, or train_own
    aristos_training_state_t train_last = {};   // what the last forward saved
    // stage stopwatch
    static constexpr int PROF_SETS = 64;      // ring of event sets: stage times average over the last 64 forwards
    static constexpr int PROF_EVENTS = 8;     // per set: 5 stage boundaries, "rows sent", "counts arrived", "GEMMs done"
    bool profiling = false;
    int64_t prof_n = 0;
    std::vector<cudaEvent_t> ev_prof;         // [PROF_SETS][PROF_EVENTS]; 5-7 are marked by the direct exchange only
    bool prof_exchange = false;               // the last forward marked events 6 and 7
    bool prof_sent = false;                   // this forward recorded event 5
};

namespace {

struct Carver {
    size_t off = 0;
    size_t take(size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 1024);
        return o;
    }
};

// Saved routing of one forward: [topk_idx | topk_w | slot_of | load-balance statistics], each part 256-byte aligned.
size_t training_bytes(const aristos_moe* L) {
    const size_t sk = align_up((size_t)L->S * L->k * 4, 256);
    return 3 * sk + aristos_load_balance_stats_bytes(L->E);
}

// Lays the buffers out; with base == nullptr only the total size is computed.
size_t plan_workspace(aristos_moe* L, char* base) {
    Carver c;
    const size_t S = L->S, k = L->k, E = L->E, cap = L->cap, H = L->H, I = L->I, elt = L->elt;
    const size_t rows_local = (size_t)L->groups * cap;   // rows this rank's experts may receive
#define CARVE(field, type, bytes)                                   \
    {                                                               \
        const size_t o = c.take(bytes);                             \
        if (base) L->field = reinterpret_cast<type>(base + o);      \
    }
    CARVE(dev_status, int32_t*, 4)
    CARVE(topk_idx, int32_t*, S * k * 4)
    CARVE(topk_w, float*, S * k * 4)
    CARVE(count, int32_t*, E * 4)
    CARVE(rcount, int32_t*, (size_t)L->groups * 4)
    CARVE(ffn_done, int32_t*, L->ffn_done_ints * 4)
    if (L->dense) {
        CARVE(send_base, int32_t*, E * 4)
        CARVE(dense_count, int32_t*, (size_t)L->E_local * 4)
        CARVE(src_off, int32_t*, (size_t)L->E_local * (L->world + 1) * 4)
    }
    CARVE(slot_of, int32_t*, S * k * 4)
    CARVE(token_of_slot, int32_t*, E * cap * 4)
    CARVE(gate_bias, float*, E * 4)
    if (L->cfg.is_training) CARVE(train_own, void*, training_bytes(L))
    CARVE(dispatch_scratch, void*, L->dispatch_scratch_bytes)
    if (L->gate_scratch_bytes) CARVE(gate_scratch, void*, L->gate_scratch_bytes)
    if (L->fp8) {
        CARVE(xq, void*, S * H)
        CARVE(sx, float*, S * (H / 128) * 4)
        if (L->world == 1) {
            CARVE(xgq, void*, E * cap * H)
            CARVE(sxg, float*, E * cap * (H / 128) * 4)
        }
        CARVE(hq, void*, rows_local * I)
        CARVE(sh, float*, rows_local * (I / 128) * 4)
    } else {
        CARVE(xg, void*, E * cap * H * elt)
    }
    CARVE(h, void*, rows_local * I * elt)
    CARVE(yr, void*, rows_local * H * elt)
    if (L->world > 1 && !L->p2p) {
        CARVE(xr, void*, rows_local * H * elt)
        CARVE(yg, void*, E * cap * H * elt)
    } else if (base && L->p2p) {
        // the peers write straight into this rank's exchange region
        L->xr = ep_p2p_xr(L->p2p);
        L->yg = ep_p2p_yg(L->p2p);
        L->rcount = ep_p2p_rcount(L->p2p);
        if (L->fp8) {      // the quantised rows and their scales arrive here from every rank
            L->xgq = L->xr;
            L->sxg = static_cast<float*>(ep_p2p_aux(L->p2p));
        }
    } else if (base) {
        L->xr = L->xg;
        L->yg = L->yr;
    }
    for (int i = 0; i < aristos_moe::HOST_SLOTS; ++i) {
        CARVE(slots[i].x_dev, void*, S * H * elt)
        CARVE(slots[i].out_dev, void*, S * H * elt)
    }
#undef CARVE
    return c.off;
}

// Waits for `ev` with the layer's wall-clock limit when the layer takes part in an exchange (a peer that stops leaves
// stream waits and flag waits unsatisfied; cudaEventSynchronize / cudaDeviceSynchronize would then never return).
// On expiry this rank's own flag words are set to the current epoch from the host, which completes every wait of
// the forward in flight; the forward's result is then undefined, the handle is marked failed and
// ARISTOS_ERR_DEVICE_TIMEOUT returned. The NCCL transport has no flags to release: the handle is marked failed and
// the caller has to end the process group.
aristos_status_t wait_event_bounded(aristos_moe* L, cudaEvent_t ev) {
    if (L->world == 1 || !ev) {
        if (ev) ARISTOS_CUDA_TRY(cudaEventSynchronize(ev));
        return ARISTOS_OK;
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (int spins = 0;; ++spins) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return ARISTOS_OK;
        if (q != cudaErrorNotReady) return cuda_fail(q, "cudaEventQuery");
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > L->timeout_ms) break;
        if (spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    L->failed = true;
    if (L->p2p) {
        ARISTOS_TRY(ep_p2p_release_local_waits(L->p2p));
        // the released forward now runs to its end on whatever rows are there; its bounded kernels cannot hang
        ARISTOS_CUDA_TRY(cudaEventSynchronize(ev));
        set_last_error("a peer did not take part in the exchange within %d ms: this rank's waits were released, the "
                       "forward's result is undefined", L->timeout_ms);
    } else {
        set_last_error("the NCCL exchange did not complete within %d ms", L->timeout_ms);
    }
    return ARISTOS_ERR_DEVICE_TIMEOUT;
}

aristos_status_t ensure_workspace(aristos_moe* L) {
    if (L->ws) return ARISTOS_OK;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, L->ws_bytes);
    if (e != cudaSuccess) {
        set_last_error("cudaMalloc of the %zu-byte layer workspace failed: %s", L->ws_bytes, cudaGetErrorString(e));
        return ARISTOS_ERR_NOMEM;
    }
    L->ws = p;
    L->ws_owned = true;
    plan_workspace(L, static_cast<char*>(p));
    ARISTOS_CUDA_TRY(cudaMemset(L->dev_status, 0, 4));
    L->bias_ready = false;
    return ARISTOS_OK;
}

}  // namespace

extern "C" {

aristos_status_t aristos_moe_create(const aristos_config_t* cfg, int rank, int world, const void* nccl_unique_id,
                                    aristos_moe_t** out) {
    if (!cfg || !out) return ARISTOS_ERR_INVALID_ARG;
    ARISTOS_TRY(aristos_config_validate(cfg));
    if (world < 1 || rank < 0 || rank >= world) { set_last_error("create: bad rank/world"); return ARISTOS_ERR_INVALID_ARG; }
    if (cfg->ep_world != world) { set_last_error("create: config ep_world (%d) != world (%d)", cfg->ep_world, world); return ARISTOS_ERR_CONFIG; }
    if (world > 1 && !nccl_unique_id) { set_last_error("create: world > 1 needs a NCCL unique id"); return ARISTOS_ERR_INVALID_ARG; }
    if (cfg->torch_dtype == ARISTOS_DTYPE_FP8_E4M3) {
        const char* tr = getenv("ARISTOS_EP_TRANSPORT");
        if (world > 1 && tr && !strcmp(tr, "nccl")) {
            set_last_error("create: torch_dtype 4 (fp8) across ranks needs the peer-memory transport");
            return ARISTOS_ERR_UNSUPPORTED;
        }
        if (cfg->hidden_size % 512 != 0 || cfg->intermediate_size % 128 != 0) {
            set_last_error("create: fp8 needs hidden_size %% 512 == 0 and intermediate_size %% 128 == 0");
            return ARISTOS_ERR_CONFIG;
        }
    }
    int dev = 0;
    ARISTOS_CUDA_TRY(cudaGetDevice(&dev));
    aristos_moe* L = new (std::nothrow) aristos_moe();
    if (!L) return ARISTOS_ERR_NOMEM;
    L->cfg = *cfg;
    L->rank = rank;
    L->world = world;
    L->device = dev;
    L->S = aristos_config_tokens(cfg);
    L->H = cfg->hidden_size;
    L->I = cfg->intermediate_size;
    L->E = cfg->num_experts;
    L->k = cfg->expert_top_k;
    L->cap = aristos_config_capacity(cfg);
    L->E_local = L->E / world;
    L->groups = L->E_local * world;
    L->fp8 = cfg->torch_dtype == ARISTOS_DTYPE_FP8_E4M3;
    L->elt = L->fp8 ? 2 : dtype_bytes(cfg->torch_dtype);     // fp8: activations and output are bf16
    if ((int64_t)L->E * L->cap > 0x7fffffffLL) { delete L; set_last_error("create: E*capacity overflows int32"); return ARISTOS_ERR_CONFIG; }
    if (L->groups > 1024) { delete L; set_last_error("create: more than 1024 row groups per rank"); return ARISTOS_ERR_CONFIG; }
    L->dispatch_scratch_bytes = aristos_dispatch_scratch_bytes(L->S, L->k, L->E);
    L->ffn_done_ints = (size_t)L->groups * ((L->cap + 127) / 128);
    {
        // many experts, 16-bit inputs: the gate screens on the tensor cores (ARISTOS_GATE=exact keeps the
        // all-experts kernel)
        const int gdt = L->fp8 ? ARISTOS_DTYPE_BF16 : L->cfg.torch_dtype;
        const char* g = getenv("ARISTOS_GATE");
        // it pays when few of the experts can reach the top k: measured 0.19 -> 0.07 ms for 8192 tokens, 128 experts,
        // top-4, but 0.08 -> 0.15 ms for 4096 tokens, 32 experts, top-8
        const bool screen = (gdt == ARISTOS_DTYPE_BF16 || gdt == ARISTOS_DTYPE_F16) && L->E >= 64 && L->E <= 256 &&
                            L->E % 4 == 0 && L->E >= 8 * L->k && !(g && !strcmp(g, "exact"));
        L->gate_scratch_bytes = screen ? aristos_gate_scratch_bytes(L->S, L->E) : 0;
    }
    if (world > 1) {
        // SMs handed to NCCL's copy kernels while the persistent GEMM grid runs on the rest
        int nccl_ctas = 8;
        if (const char* env = getenv("ARISTOS_EP_NCCL_CTAS")) nccl_ctas = atoi(env);
        aristos_status_t s = ep_comm_create(nccl_unique_id, rank, world, nccl_ctas, &L->comm);
        if (s != ARISTOS_OK) { delete L; return s; }
        cudaError_t e = cudaStreamCreateWithFlags(&L->comm_stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_dispatched, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_returned, cudaEventDisableTiming);
        // row windows of the overlapped exchange
        ep_row_windows(L->cap, 4, 512, &L->chunk_rows, &L->chunks);
        if (const char* env = getenv("ARISTOS_EP_CHUNKS"))
            if (atoi(env) >= 1) ep_row_windows(L->cap, std::min(atoi(env), EP_MAX_WINDOWS), 128, &L->chunk_rows, &L->chunks);
        if (const char* env = getenv("ARISTOS_EP_TIMEOUT_MS"))
            if (atoi(env) >= 1) L->timeout_ms = atoi(env);
        L->ffn_sm_limit = device_sm_count() - (nccl_ctas > 0 ? nccl_ctas : 16);
        if (const char* env = getenv("ARISTOS_EP_FFN_SMS"))
            if (atoi(env) >= 1) L->ffn_sm_limit = atoi(env);
        L->ev_in.resize(L->chunks);
        L->ev_out.resize(L->chunks);
        for (int c = 0; c < L->chunks && e == cudaSuccess; ++c) {
            e = cudaEventCreateWithFlags(&L->ev_in[c], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_out[c], cudaEventDisableTiming);
        }
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_last, cudaEventDisableTiming);
        if (e != cudaSuccess) { aristos_moe_destroy(L); return cuda_fail(e, "stream/event creation"); }
        // transport of the rows: peer memory (default) or NCCL send/recv (ARISTOS_EP_TRANSPORT=nccl, or when the
        // peer-memory set-up is not possible on this machine)
        const char* tr = getenv("ARISTOS_EP_TRANSPORT");
        if (!(tr && !strcmp(tr, "nccl")) && L->chunks <= EP_MAX_WINDOWS) {
            const size_t block_bytes = (size_t)L->cap * L->H * L->elt;
            // fp8: received rows are e4m3 codes (one byte) plus one fp32 scale per 128 elements; outputs stay bf16
            const size_t in_bytes = L->fp8 ? (size_t)L->groups * L->cap * L->H : (size_t)L->groups * block_bytes;
            const size_t aux_bytes = L->fp8 ? (size_t)L->groups * L->cap * (L->H / 128) * 4 : 0;
            aristos_status_t ps = ep_p2p_create(L->comm, rank, world, L->groups, in_bytes, (size_t)L->E * block_bytes,
                                                aux_bytes, &L->p2p);
            if (ps == ARISTOS_OK) {
                L->ffn_sm_limit = 0;      // nothing else needs SMs while rows travel
                // default: the gather / return kernels store through peer pointers; ARISTOS_EP_MODE=windows selects
                // the copy-engine pipeline over padded row windows instead
                const char* mode = getenv("ARISTOS_EP_MODE");
                L->ep_direct = !(mode && !strcmp(mode, "windows"));
                // one window by default: on two GPUs, splitting the GEMMs to hide the transfers behind them was
                // no faster (10.5, 10.5, 10.8 ms of device time for 1, 2, 4 windows: 16384 tokens per rank, 8 experts,
                // H 4096, I 14336)
                L->direct_windows = 1;
                if (const char* env = getenv("ARISTOS_EP_DIRECT_WINDOWS"))
                    if (atoi(env) >= 1) L->direct_windows = atoi(env);
                L->direct_windows = std::min(L->direct_windows, (int)L->ev_out.size());
                // the tensor-core GEMM returns its output tiles itself (TMA stores through peer mappings);
                // ARISTOS_EP_FUSED_RETURN=0 keeps the separate return kernel
                const char* fr = getenv("ARISTOS_EP_FUSED_RETURN");
                const int tdt = cfg->torch_dtype;
                const bool tc = tdt == ARISTOS_DTYPE_BF16 || tdt == ARISTOS_DTYPE_F16 || tdt == ARISTOS_DTYPE_TF32;
                L->fused_return = world <= 8 && !(fr && !strcmp(fr, "0")) && (L->fp8 || (L->ep_direct && tc));
                // the tensor-core up projection waits for each source rank's rows itself (own rows first) instead
                // of the stream waiting for every rank before the first tile; ARISTOS_EP_KERNEL_WAIT=0 keeps the
                // stream waits
                // fp8: the rows an expert receives from all ranks are packed into one group (whole tiles of one
                // expert instead of one padded group per (source, expert)); ARISTOS_EP_DENSE=0 keeps the groups apart
                const char* dn = getenv("ARISTOS_EP_DENSE");
                L->dense = L->fp8 && L->fused_return && !(dn && !strcmp(dn, "0"));
                const char* kw = getenv("ARISTOS_EP_KERNEL_WAIT");
                L->kernel_wait = L->ep_direct && tc && !(kw && !strcmp(kw, "0"));
                // ... and then only the rows a rank keeps are gathered before its up projection starts; the rows for
                // the other ranks leave on the communication stream while the tensor cores work on the local rows
                // (ARISTOS_EP_OVERLAP_GATHER=0: the whole gather runs first)
                const char* og = getenv("ARISTOS_EP_OVERLAP_GATHER");
                L->overlap_gather = L->kernel_wait && L->direct_windows == 1 && !(og && !strcmp(og, "0"));
            }
            else if (L->fp8 || (tr && !strcmp(tr, "p2p")) || ps != ARISTOS_ERR_UNSUPPORTED) {
                // ARISTOS_ERR_UNSUPPORTED is the agreed answer of every rank (all fall back to NCCL together); any
                // other status means the bootstrap itself failed
                aristos_moe_destroy(L);
                return ps;
            }
        }
    }
    L->ws_bytes = plan_workspace(L, nullptr);
    *out = L;
    return ARISTOS_OK;
}

size_t aristos_moe_workspace_bytes(const aristos_moe_t* L) { return L ? L->ws_bytes : 0; }

aristos_status_t aristos_moe_set_bias(aristos_moe_t* L, const void* b1, const void* b3, const void* b2) {
    if (!L) return ARISTOS_ERR_INVALID_ARG;
    if (L->fp8 && (b1 || b3 || b2)) {
        set_last_error("set_bias: the fp8 expert FFN has no bias epilogue");
        return ARISTOS_ERR_UNSUPPORTED;
    }
    if ((b1 && !aligned16(b1)) || (b3 && !aligned16(b3)) || (b2 && !aligned16(b2))) {
        set_last_error("set_bias: pointers must be 16-byte aligned");
        return ARISTOS_ERR_INVALID_ARG;
    }
    L->b1 = b1;
    L->b3 = b3;
    L->b2 = b2;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_set_workspace(aristos_moe_t* L, void* workspace, size_t bytes) {
    if (!L || !workspace) return ARISTOS_ERR_INVALID_ARG;
    if (bytes < L->ws_bytes) { set_last_error("workspace: %zu bytes given, %zu needed", bytes, L->ws_bytes); return ARISTOS_ERR_WORKSPACE; }
    if (reinterpret_cast<uintptr_t>(workspace) % 1024 != 0) { set_last_error("workspace must be 1024-byte aligned"); return ARISTOS_ERR_INVALID_ARG; }
    if (L->ws && L->ws_owned) cudaFree(L->ws);
    L->ws = workspace;
    L->ws_owned = false;
    plan_workspace(L, static_cast<char*>(workspace));
    ARISTOS_CUDA_TRY(cudaMemset(L->dev_status, 0, 4));
    L->bias_ready = false;
    return ARISTOS_OK;
}

static aristos_status_t forward_impl(aristos_moe_t* L, const void* x, const void* w_gate, const float* gate_bias,
                                     const void* w1, const void* w3, const void* w2, const void* scales, void* out,
                                     void* stream, bool* exchange_started);

aristos_status_t aristos_moe_forward(aristos_moe_t* L, const void* x, const void* w_gate, const float* gate_bias,
                                     const void* w1, const void* w3, const void* w2, const void* scales, void* out,
                                     void* stream) {
    if (!L || !x || !w_gate || !w1 || !w2 || !out) { set_last_error("forward: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    if (L->cfg.hidden_act == ARISTOS_ACT_SWIGLU && !w3) { set_last_error("forward: SwiGLU needs w3"); return ARISTOS_ERR_INVALID_ARG; }
    if (L->fp8 && !scales) { set_last_error("forward: fp8 needs the weight scales"); return ARISTOS_ERR_INVALID_ARG; }
    if (L->failed) {
        set_last_error("forward: an earlier forward of this expert-parallel layer failed or timed out; its exchange "
                       "epochs no longer match the peers' - destroy the layer on every rank and create it again");
        return ARISTOS_ERR_DEVICE_TIMEOUT;
    }
    ARISTOS_TRY(ensure_workspace(L));
    bool exchange_started = false;
    const aristos_status_t s = forward_impl(L, x, w_gate, gate_bias, w1, w3, w2, scales, out, stream, &exchange_started);
    // a forward that stopped after it announced a new epoch leaves this rank out of step with its peers
    if (s != ARISTOS_OK && exchange_started) L->failed = true;
    if (s == ARISTOS_OK && L->ev_last) {
        if (cudaEventRecord(L->ev_last, static_cast<cudaStream_t>(stream)) == cudaSuccess) L->ev_last_valid = true;
    }
    return s;
}

static aristos_status_t forward_impl(aristos_moe_t* L, const void* x, const void* w_gate, const float* gate_bias,
                                     const void* w1, const void* w3, const void* w2, const void* scales, void* out,
                                     void* stream, bool* exchange_started) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t launches0 = launch_counter();
    const int dt = L->fp8 ? ARISTOS_DTYPE_BF16 : L->cfg.torch_dtype;     // dtype of x, out and the expert outputs

    const float* bias = gate_bias;
    if (!bias && L->cfg.gate_bias_zipf_s > 0.0) {
        if (!L->bias_ready) {
            std::vector<float> b(L->E);
            aristos_zipf_bias_host(b.data(), L->E, L->cfg.gate_bias_zipf_s);
            ARISTOS_CUDA_TRY(cudaMemcpyAsync(L->gate_bias, b.data(), sizeof(float) * L->E, cudaMemcpyHostToDevice, st));
            ARISTOS_CUDA_TRY(cudaStreamSynchronize(st));   // b goes out of scope
            L->bias_ready = true;
        }
        bias = L->gate_bias;
    }

    const int prof_set = (int)(L->prof_n % aristos_moe::PROF_SETS) * aristos_moe::PROF_EVENTS;
    L->prof_sent = false;
    L->prof_exchange = false;
#define PROF_MARK(i) do { if (L->profiling) ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_prof[prof_set + i], st)); } while (0)
    // NVTX ranges (host side: they bracket the enqueue of each stage, so a profiler timeline groups the stage's
    // launches; the reference links NVTX without calling it, CMakeLists.txt:104-118)
    struct StageRange {
        bool open = false;
        void next(const char* name) {
            if (open) nvtxRangePop();
            nvtxRangePushA(name);
            open = true;
        }
        ~StageRange() { if (open) nvtxRangePop(); }
    };
    StageRange whole, stage;
    whole.next("aristos_moe_forward");
    PROF_MARK(0);
    stage.next("gate");
    ARISTOS_TRY(aristos_gate_topk_screened(x, w_gate, bias, L->S, L->H, L->E, L->k, L->cfg.gate_fn, L->cfg.renorm_topk,
                                           dt, L->topk_idx, L->topk_w, L->gate_scratch_bytes ? L->gate_scratch : nullptr,
                                           L->gate_scratch_bytes, L->dev_status, st));
    PROF_MARK(1);
    stage.next("dispatch");
    ARISTOS_TRY(dispatch_impl(L->topk_idx, L->S, L->k, L->E, L->cap, L->count, L->slot_of, L->token_of_slot,
                              L->dispatch_scratch, L->dispatch_scratch_bytes, L->dev_status, st));
    if (L->cfg.is_training) {
        // training mode: the routing of this forward is copied out of the working buffers (which the next forward
        // overwrites) together with its load-balance statistics
        char* tb = static_cast<char*>(L->train_buf ? L->train_buf : L->train_own);
        const size_t skb = (size_t)L->S * L->k * 4, sk = align_up(skb, 256);
        aristos_training_state_t ts;
        ts.topk_idx = reinterpret_cast<int32_t*>(tb);
        ts.topk_w = reinterpret_cast<float*>(tb + sk);
        ts.slot_of = reinterpret_cast<int32_t*>(tb + 2 * sk);
        ts.load_balance = reinterpret_cast<float*>(tb + 3 * sk);
        ts.tokens = L->S;
        ts.top_k = L->k;
        ts.num_experts = L->E;
        ARISTOS_CUDA_TRY(cudaMemcpyAsync(const_cast<int32_t*>(ts.topk_idx), L->topk_idx, skb, cudaMemcpyDeviceToDevice, st));
        ARISTOS_CUDA_TRY(cudaMemcpyAsync(const_cast<float*>(ts.topk_w), L->topk_w, skb, cudaMemcpyDeviceToDevice, st));
        ARISTOS_CUDA_TRY(cudaMemcpyAsync(const_cast<int32_t*>(ts.slot_of), L->slot_of, skb, cudaMemcpyDeviceToDevice, st));
        ARISTOS_TRY(aristos_load_balance_stats(L->topk_idx, L->topk_w, L->slot_of, L->S, L->k, L->E,
                                               const_cast<float*>(ts.load_balance), stream));
        L->train_last = ts;
    }
    const size_t nb1 = (size_t)L->E_local * (L->I / 128) * (L->H / 128);
    const bool swiglu = L->cfg.hidden_act == ARISTOS_ACT_SWIGLU;
    const float* s1 = static_cast<const float*>(scales);
    const float* s3 = (L->fp8 && swiglu) ? s1 + nb1 : nullptr;
    const float* s2 = L->fp8 ? s1 + nb1 * (swiglu ? 2 : 1) : nullptr;
    if (L->fp8 && L->world == 1) {
        // quantise the tokens per row and 128 elements, then gather codes and scales into expert-major order
        ARISTOS_TRY(aristos_quantize_fp8(x, 1, L->S, L->H, 1, ARISTOS_DTYPE_BF16, L->xq, L->sx, stream));
        ARISTOS_TRY(aristos_permute(L->xq, L->slot_of, L->S, L->k, L->H, ARISTOS_DTYPE_FP8_E4M3, L->xgq, st));
        ARISTOS_TRY(aristos_permute(L->sx, L->slot_of, L->S, L->k, L->H / 128, ARISTOS_DTYPE_F32, L->sxg, st));
    } else if (L->fp8) {
        // expert parallel: the gather stores every kept row (codes and scales) straight into the owner's memory, so
        // only rows that exist cross NVLink (capacity = tokens would make padded blocks enormous)
        PeerPtrs rows_dst, scales_dst, y_dst;
        ep_p2p_peer_ptrs(L->p2p, EP_BUF_XR, rows_dst.p);
        ep_p2p_peer_ptrs(L->p2p, EP_BUF_AUX, scales_dst.p);
        ep_p2p_peer_ptrs(L->p2p, EP_BUF_YG, y_dst.p);
        ep_p2p_begin(L->p2p);
        *exchange_started = true;
        stage.next("exchange");
        if (L->dense) {
            // every rank learns every rank's counts first (one small kernel + flag), then knows where its rows start
            // inside each expert's dense group at the owner
            ARISTOS_TRY(ep_p2p_send_counts(L->p2p, L->count, L->E, L->E_local, st, /*to_all=*/true));
        }
        ARISTOS_TRY(aristos_quantize_fp8(x, 1, L->S, L->H, 1, ARISTOS_DTYPE_BF16, L->xq, L->sx, stream));
        if (L->dense) {
            const int dense_rows = L->world * L->cap;          // rows of one expert's group: all sources, worst case
            ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_COUNT, 0, st));
            ARISTOS_TRY(dense_exchange_plan(ep_p2p_allcount(L->p2p), L->world, L->E, L->E_local, L->rank, L->send_base,
                                            L->dense_count, L->src_off, st));
            ARISTOS_TRY(permute_rows_to_peers(L->xq, L->slot_of, L->S, L->k, (size_t)L->H, L->E_local, L->cap, L->rank, 0,
                                              L->cap, rows_dst, st, nullptr, 0, nullptr, L->send_base, dense_rows));
            ARISTOS_TRY(permute_rows_to_peers(L->sx, L->slot_of, L->S, L->k, (size_t)(L->H / 128) * 4, L->E_local, L->cap,
                                              L->rank, 0, L->cap, scales_dst, st, nullptr, 0, nullptr, L->send_base,
                                              dense_rows));
            ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_IN, 0, st));
            PROF_MARK(2);
            ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_IN, 0, st));
            stage.next("expert_ffn");
            if (swiglu && !w3) { set_last_error("forward: SwiGLU needs w3"); return ARISTOS_ERR_INVALID_ARG; }
            ARISTOS_TRY(expert_ffn_fp8_sm100(L->xgq, L->sxg, L->dense_count, L->E_local, dense_rows, L->E_local, w1, s1, w3,
                                             s3, w2, s2, L->h, L->hq, L->sh, L->yr, L->H, L->I, L->cfg.hidden_act, 0,
                                             dense_rows, 0, L->dev_status, st, y_dst.p, L->world, L->rank, L->src_off,
                                             L->cap));
        } else {
        PeerPtrs count_dst;
        ep_p2p_peer_ptrs(L->p2p, EP_BUF_RCOUNT, count_dst.p);
        ARISTOS_TRY(permute_rows_to_peers(L->xq, L->slot_of, L->S, L->k, (size_t)L->H, L->E_local, L->cap, L->rank, 0,
                                          L->cap, rows_dst, st, L->count, L->E, &count_dst));
        ARISTOS_TRY(permute_rows_to_peers(L->sx, L->slot_of, L->S, L->k, (size_t)(L->H / 128) * 4, L->E_local, L->cap,
                                          L->rank, 0, L->cap, scales_dst, st));
        ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_IN, 0, st));
        PROF_MARK(2);
        ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_IN, 0, st));
        stage.next("expert_ffn");
        if (L->fused_return) {
            // the down projection stores its valid output rows straight into the ranks they came from
            if (swiglu && !w3) { set_last_error("forward: SwiGLU needs w3"); return ARISTOS_ERR_INVALID_ARG; }
            ARISTOS_TRY(expert_ffn_fp8_sm100(L->xgq, L->sxg, L->rcount, L->groups, L->cap, L->E_local, w1, s1, w3, s3, w2,
                                             s2, L->h, L->hq, L->sh, L->yr, L->H, L->I, L->cfg.hidden_act, 0, L->cap, 0,
                                             L->dev_status, st, y_dst.p, L->world, L->rank));
        } else {
            ARISTOS_TRY(aristos_expert_ffn_fp8(L->xgq, L->sxg, L->rcount, L->groups, L->cap, L->E_local, w1, s1, w3, s3,
                                               w2, s2, L->h, L->hq, L->sh, L->yr, L->H, L->I, L->cfg.hidden_act, 0,
                                               L->cap, 0, L->dev_status, st));
            ARISTOS_TRY(return_rows_to_peers(L->yr, L->rcount, L->groups, L->E_local, L->cap, (size_t)L->H * 2, L->rank,
                                             0, L->cap, y_dst, st));
        }
        }
        ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_RET, 0, st));
        ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_RET, 0, st));
    } else if (!(L->p2p && L->ep_direct)) {
        ARISTOS_TRY(aristos_permute(x, L->slot_of, L->S, L->k, L->H, dt, L->xg, st));
    }
    if (!(L->fp8 && L->world > 1)) PROF_MARK(2);
    if (!(L->fp8 && L->world > 1)) stage.next(L->world > 1 ? "exchange+expert_ffn" : "expert_ffn");

    if (L->fp8 && L->world > 1) {
        // done above
    } else if (L->fp8) {
        ARISTOS_TRY(aristos_expert_ffn_fp8(L->xgq, L->sxg, L->count, L->E, L->cap, L->E, w1, s1, w3, s3, w2, s2, L->h,
                                           L->hq, L->sh, L->yr, L->H, L->I, L->cfg.hidden_act, 0, L->cap, 0,
                                           L->dev_status, st));
    } else if (L->world == 1 && (dt == ARISTOS_DTYPE_BF16 || dt == ARISTOS_DTYPE_F16 || dt == ARISTOS_DTYPE_TF32)) {
        FfnEpArgs extra;                     // no exchange; the scratch lets small row groups run as one launch
        extra.updown_scratch = L->ffn_done;
        extra.updown_scratch_ints = L->ffn_done_ints;
        const int fmt = dt == ARISTOS_DTYPE_BF16 ? 0 : (dt == ARISTOS_DTYPE_F16 ? 1 : 2);
        ARISTOS_TRY(expert_ffn_tc_sm100(L->xg, L->count, L->E, L->cap, L->E, w1, w3, w2, L->b1, L->b3, L->b2, L->h, L->yr,
                                        L->H, L->I, L->cfg.hidden_act, fmt, 0, L->cap, 0, L->dev_status, st, &extra));
    } else if (L->world == 1) {
        ARISTOS_TRY(aristos_expert_ffn_bias(L->xg, L->count, L->E, L->cap, L->E, w1, w3, w2, L->b1, L->b3, L->b2, L->h, L->yr, L->H, L->I,
                                       L->cfg.hidden_act, dt, 0, L->cap, 0, L->dev_status, st));
    } else if (L->p2p && L->ep_direct) {
        // the gather IS the dispatch all-to-all: every kept row is stored straight into its expert's rank, the expert
        // outputs come back the same way; only rows that exist travel. With one row window everything stays on the caller's stream; with more, the light gather / return
        // kernels run on the communication stream and share the SMs with the persistent GEMM grid, window by window.
        PeerPtrs rows_dst, y_dst;
        ep_p2p_peer_ptrs(L->p2p, EP_BUF_XR, rows_dst.p);
        ep_p2p_peer_ptrs(L->p2p, EP_BUF_YG, y_dst.p);
        const size_t row_bytes = (size_t)L->H * L->elt;
        const int nwin = L->direct_windows;
        const int win_rows = ceil_div(ceil_div(L->cap, nwin), 256) * 256;
        const bool overlap = L->overlap_gather && nwin == 1;
        cudaStream_t cs = (nwin > 1 || overlap) ? L->comm_stream : st;
        ep_p2p_begin(L->p2p);
        *exchange_started = true;
        // the row counts go first, with a flag of their own: every rank can build its tile list as soon as its peers
        // have routed their tokens, long before their rows have all arrived
        ARISTOS_TRY(ep_p2p_send_counts(L->p2p, L->count, L->E, L->E_local, st));
        if (overlap)      // the rows this rank keeps: a local copy, complete before the up projection is launched
            ARISTOS_TRY(permute_rows_to_peers(x, L->slot_of, L->S, L->k, row_bytes, L->E_local, L->cap, L->rank, 0, L->cap,
                                              rows_dst, st, nullptr, 0, nullptr, nullptr, 0, /*dest_filter=*/1));
        if (cs != st) {
            ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_dispatched, st));
            ARISTOS_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_dispatched, 0));
        }
        for (int c = 0; c < nwin; ++c) {
            const int r0 = c * win_rows, r1 = std::min(L->cap, r0 + win_rows);
            if (r0 >= r1) break;
            ARISTOS_TRY(permute_rows_to_peers(x, L->slot_of, L->S, L->k, row_bytes, L->E_local, L->cap, L->rank, r0, r1,
                                              rows_dst, cs, nullptr, 0, nullptr, nullptr, 0, overlap ? 2 : 0));
            ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_IN, c, cs));
        }
        if (L->profiling) {          // "rows sent": the gather kernels and their flags are behind this event
            ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_prof[prof_set + 5], cs));
            L->prof_sent = true;
        }
        if (overlap) ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_in[0], cs));      // joined before the combine
        ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_COUNT, 0, st));
        PROF_MARK(6);                // every rank's counts are here
        const bool tc = dt == ARISTOS_DTYPE_BF16 || dt == ARISTOS_DTYPE_F16 || dt == ARISTOS_DTYPE_TF32;
        for (int c = 0; c < nwin; ++c) {
            const int r0 = c * win_rows, r1 = std::min(L->cap, r0 + win_rows);
            if (r0 >= r1) break;
            // either the stream waits for the rows of every rank, or the up projection waits per source rank while
            // it already works on the rows that are there (its own first)
            if (!(L->kernel_wait && tc)) ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_IN, c, st));
            if (tc) {
                FfnEpArgs ep;
                ep.first_source = L->rank;
                if (overlap) ep.self_source = L->rank;
                if (nwin == 1) {             // one row window: small row groups run both projections as one launch
                    ep.updown_scratch = L->ffn_done;
                    ep.updown_scratch_ints = L->ffn_done_ints;
                }
                if (L->kernel_wait) {
                    ep.src_flags = ep_p2p_flags(L->p2p, EP_FLAG_IN, c);
                    ep.flag_epoch = ep_p2p_epoch(L->p2p);
                    ep.flag_limit_ms = 2000;
                }
                if (L->fused_return) {
                    // the epilogue of the down projection IS the return all-to-all: each output tile is stored into
                    // the buffer of the rank its rows came from while the tensor cores work on the next tile
                    ep.peer_y = y_dst.p;
                    ep.peer_world = L->world;
                    ep.peer_rank = L->rank;
                }
                const int fmt = dt == ARISTOS_DTYPE_BF16 ? 0 : (dt == ARISTOS_DTYPE_F16 ? 1 : 2);
                ARISTOS_TRY(expert_ffn_tc_sm100(L->xr, L->rcount, L->groups, L->cap, L->E_local, w1, w3, w2, L->b1, L->b3,
                                                L->b2, L->h, L->yr, L->H, L->I, L->cfg.hidden_act, fmt, r0, r1, 0,
                                                L->dev_status, st, &ep));
                if (L->fused_return) {
                    ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_RET, c, st));
                    continue;
                }
            } else {
                ARISTOS_TRY(aristos_expert_ffn_bias(L->xr, L->rcount, L->groups, L->cap, L->E_local, w1, w3, w2, L->b1,
                                                    L->b3, L->b2, L->h, L->yr, L->H, L->I, L->cfg.hidden_act, dt, r0, r1,
                                                    0, L->dev_status, st));
            }
            if (cs != st) {
                ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_out[c], st));
                ARISTOS_CUDA_TRY(cudaStreamWaitEvent(cs, L->ev_out[c], 0));
            }
            ARISTOS_TRY(return_rows_to_peers(L->yr, L->rcount, L->groups, L->E_local, L->cap, row_bytes, L->rank, r0, r1,
                                             y_dst, cs));
            ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_RET, c, cs));
        }
        PROF_MARK(7);                // this rank's GEMMs (and, fused, its return stores and flags) are done
        L->prof_exchange = L->profiling;
        for (int c = 0; c < nwin; ++c)
            if (c * win_rows < L->cap) ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_RET, c, st));
        // the gather for the other ranks still reads x and the routing tensors: the caller's stream joins it
        if (overlap) ARISTOS_CUDA_TRY(cudaStreamWaitEvent(st, L->ev_in[0], 0));
    } else if (L->p2p) {
        // rows are pushed into the destination GPUs by the copy engines; flags + stream waits order the streams
        const size_t row_bytes = (size_t)L->H * L->elt;
        const size_t block_stride = (size_t)L->cap * row_bytes;
        ep_p2p_begin(L->p2p);
        *exchange_started = true;
        ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_dispatched, st));
        ARISTOS_CUDA_TRY(cudaStreamWaitEvent(L->comm_stream, L->ev_dispatched, 0));
        ARISTOS_TRY(ep_p2p_push(L->p2p, EP_FLAG_COUNT, L->count, 1, (size_t)L->E_local * 4, 0, (size_t)L->E_local * 4,
                                L->comm_stream));
        ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_COUNT, 0, L->comm_stream));
        for (int c = 0; c < L->chunks; ++c) {
            const int r0 = c * L->chunk_rows, r1 = std::min(L->cap, r0 + L->chunk_rows);
            ARISTOS_TRY(ep_p2p_push(L->p2p, EP_FLAG_IN, L->xg, L->E_local, block_stride, (size_t)r0 * row_bytes,
                                    (size_t)(r1 - r0) * row_bytes, L->comm_stream));
            ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_IN, c, L->comm_stream));
        }
        ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_COUNT, 0, st));
        for (int c = 0; c < L->chunks; ++c) {
            const int r0 = c * L->chunk_rows, r1 = std::min(L->cap, r0 + L->chunk_rows);
            ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_IN, c, st));
            ARISTOS_TRY(aristos_expert_ffn_bias(L->xr, L->rcount, L->groups, L->cap, L->E_local, w1, w3, w2, L->b1, L->b3, L->b2, L->h, L->yr,
                                           L->H, L->I, L->cfg.hidden_act, dt, r0, r1, 0, L->dev_status, st));
            ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_out[c], st));
            ARISTOS_CUDA_TRY(cudaStreamWaitEvent(L->comm_stream, L->ev_out[c], 0));
            ARISTOS_TRY(ep_p2p_push(L->p2p, EP_FLAG_RET, L->yr, L->E_local, block_stride, (size_t)r0 * row_bytes,
                                    (size_t)(r1 - r0) * row_bytes, L->comm_stream));
            ARISTOS_TRY(ep_p2p_signal(L->p2p, EP_FLAG_RET, c, L->comm_stream));
        }
        for (int c = 0; c < L->chunks; ++c) ARISTOS_TRY(ep_p2p_wait(L->p2p, EP_FLAG_RET, c, st));
    } else {
        const size_t row_bytes = (size_t)L->H * L->elt;
        const size_t block_stride = (size_t)L->cap * row_bytes;
        *exchange_started = true;
        ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_dispatched, st));
        ARISTOS_CUDA_TRY(cudaStreamWaitEvent(L->comm_stream, L->ev_dispatched, 0));
        // per-(source, local expert) row counts
        ARISTOS_TRY(ep_all_to_all_blocks(L->comm, L->count, L->rcount, 1, (size_t)L->E_local * 4, 0,
                                         (size_t)L->E_local * 4, L->comm_stream));
        for (int c = 0; c < L->chunks; ++c) {
            const int r0 = c * L->chunk_rows, r1 = std::min(L->cap, r0 + L->chunk_rows);
            ARISTOS_TRY(ep_all_to_all_blocks(L->comm, L->xg, L->xr, L->E_local, block_stride, (size_t)r0 * row_bytes,
                                             (size_t)(r1 - r0) * row_bytes, L->comm_stream));
            ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_in[c], L->comm_stream));
        }
        for (int c = 0; c < L->chunks; ++c) {
            const int r0 = c * L->chunk_rows, r1 = std::min(L->cap, r0 + L->chunk_rows);
            ARISTOS_CUDA_TRY(cudaStreamWaitEvent(st, L->ev_in[c], 0));
            ARISTOS_TRY(aristos_expert_ffn_bias(L->xr, L->rcount, L->groups, L->cap, L->E_local, w1, w3, w2, L->b1, L->b3, L->b2, L->h, L->yr,
                                           L->H, L->I, L->cfg.hidden_act, dt, r0, r1, L->ffn_sm_limit, L->dev_status,
                                           st));
            ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_out[c], st));
            ARISTOS_CUDA_TRY(cudaStreamWaitEvent(L->comm_stream, L->ev_out[c], 0));
            ARISTOS_TRY(ep_all_to_all_blocks(L->comm, L->yr, L->yg, L->E_local, block_stride, (size_t)r0 * row_bytes,
                                             (size_t)(r1 - r0) * row_bytes, L->comm_stream));
        }
        ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_returned, L->comm_stream));
        ARISTOS_CUDA_TRY(cudaStreamWaitEvent(st, L->ev_returned, 0));
    }
    PROF_MARK(3);
    stage.next("combine");
    ARISTOS_TRY(aristos_combine(L->yg, L->slot_of, L->topk_w, L->S, L->k, L->H, dt, out, st));
    PROF_MARK(4);
    if (L->profiling && !L->prof_sent) ARISTOS_CUDA_TRY(cudaEventRecord(L->ev_prof[prof_set + 5], st));
#undef PROF_MARK
    if (L->profiling) L->prof_n += 1;
    L->launches += launch_counter() - launches0;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_submit_host(aristos_moe_t* L, const void* x_host, const void* w_gate,
                                         const float* gate_bias, const void* w1, const void* w3, const void* w2,
                                         const void* scales, void* out_host, void* stream) {
    if (!L || !x_host || !out_host) { set_last_error("submit_host: NULL pointer"); return ARISTOS_ERR_INVALID_ARG; }
    ARISTOS_TRY(ensure_workspace(L));
    if (!L->h2d_stream) {
        ARISTOS_CUDA_TRY(cudaStreamCreateWithFlags(&L->h2d_stream, cudaStreamNonBlocking));
        ARISTOS_CUDA_TRY(cudaStreamCreateWithFlags(&L->d2h_stream, cudaStreamNonBlocking));
        for (auto& sl : L->slots) {
            ARISTOS_CUDA_TRY(cudaEventCreateWithFlags(&sl.h2d_done, cudaEventDisableTiming));
            ARISTOS_CUDA_TRY(cudaEventCreateWithFlags(&sl.compute_done, cudaEventDisableTiming));
            ARISTOS_CUDA_TRY(cudaEventCreateWithFlags(&sl.d2h_done, cudaEventDisableTiming));
        }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    aristos_moe::HostSlot& sl = L->slots[L->slot_next];
    L->slot_next = (L->slot_next + 1) % aristos_moe::HOST_SLOTS;
    if (sl.busy) {                       // the call that used this slot HOST_SLOTS submissions ago must have drained
        sl.busy = false;
        ARISTOS_TRY(wait_event_bounded(L, sl.d2h_done));
    }
    const size_t bytes = (size_t)L->S * L->H * L->elt;
    ARISTOS_CUDA_TRY(cudaMemcpyAsync(sl.x_dev, x_host, bytes, cudaMemcpyHostToDevice, L->h2d_stream));
    ARISTOS_CUDA_TRY(cudaEventRecord(sl.h2d_done, L->h2d_stream));
    ARISTOS_CUDA_TRY(cudaStreamWaitEvent(st, sl.h2d_done, 0));
    ARISTOS_TRY(aristos_moe_forward(L, sl.x_dev, w_gate, gate_bias, w1, w3, w2, scales, sl.out_dev, stream));
    ARISTOS_CUDA_TRY(cudaEventRecord(sl.compute_done, st));
    ARISTOS_CUDA_TRY(cudaStreamWaitEvent(L->d2h_stream, sl.compute_done, 0));
    ARISTOS_CUDA_TRY(cudaMemcpyAsync(out_host, sl.out_dev, bytes, cudaMemcpyDeviceToHost, L->d2h_stream));
    ARISTOS_CUDA_TRY(cudaEventRecord(sl.d2h_done, L->d2h_stream));
    sl.busy = true;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_wait_host(aristos_moe_t* L) {
    if (!L) return ARISTOS_ERR_INVALID_ARG;
    aristos_status_t first = ARISTOS_OK;
    for (auto& sl : L->slots)
        if (sl.busy) {
            sl.busy = false;
            const aristos_status_t s = wait_event_bounded(L, sl.d2h_done);
            if (first == ARISTOS_OK) first = s;
        }
    return first;
}

aristos_status_t aristos_moe_forward_host(aristos_moe_t* L, const void* x_host, const void* w_gate,
                                          const float* gate_bias, const void* w1, const void* w3, const void* w2,
                                          const void* scales, void* out_host, void* stream) {
    ARISTOS_TRY(aristos_moe_submit_host(L, x_host, w_gate, gate_bias, w1, w3, w2, scales, out_host, stream));
    return aristos_moe_wait_host(L);
}

aristos_status_t aristos_moe_routing(const aristos_moe_t* L, aristos_routing_t* out) {
    if (!L || !out) return ARISTOS_ERR_INVALID_ARG;
    if (!L->ws) { set_last_error("routing: no forward has run yet"); return ARISTOS_ERR_INVALID_ARG; }
    out->topk_idx = L->topk_idx;
    out->topk_w = L->topk_w;
    out->count = L->count;
    out->slot_of = L->slot_of;
    out->token_of_slot = L->token_of_slot;
    out->tokens = L->S;
    out->top_k = L->k;
    out->num_experts = L->E;
    out->capacity = L->cap;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_routing_to_host(const aristos_moe_t* L, int32_t* topk_idx_host, float* topk_w_host,
                                             int32_t* count_host, int32_t* slot_of_host,
                                             int32_t* token_of_slot_host) {
    if (!L) return ARISTOS_ERR_INVALID_ARG;
    if (!L->ws) { set_last_error("routing: no forward has run yet"); return ARISTOS_ERR_INVALID_ARG; }
    if (L->world > 1 && L->ev_last_valid) ARISTOS_TRY(wait_event_bounded(const_cast<aristos_moe_t*>(L), L->ev_last));
    ARISTOS_CUDA_TRY(cudaDeviceSynchronize());
    const size_t sk = (size_t)L->S * L->k;
    if (topk_idx_host) ARISTOS_CUDA_TRY(cudaMemcpy(topk_idx_host, L->topk_idx, sk * 4, cudaMemcpyDeviceToHost));
    if (topk_w_host) ARISTOS_CUDA_TRY(cudaMemcpy(topk_w_host, L->topk_w, sk * 4, cudaMemcpyDeviceToHost));
    if (count_host) ARISTOS_CUDA_TRY(cudaMemcpy(count_host, L->count, (size_t)L->E * 4, cudaMemcpyDeviceToHost));
    if (slot_of_host) ARISTOS_CUDA_TRY(cudaMemcpy(slot_of_host, L->slot_of, sk * 4, cudaMemcpyDeviceToHost));
    if (token_of_slot_host)
        ARISTOS_CUDA_TRY(cudaMemcpy(token_of_slot_host, L->token_of_slot, (size_t)L->E * L->cap * 4, cudaMemcpyDeviceToHost));
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_status(aristos_moe_t* L) {
    if (!L) return ARISTOS_ERR_INVALID_ARG;
    if (L->world > 1 && L->ev_last_valid) ARISTOS_TRY(wait_event_bounded(L, L->ev_last));
    ARISTOS_CUDA_TRY(cudaDeviceSynchronize());
    if (!L->ws) return ARISTOS_OK;
    int32_t bits = 0;
    ARISTOS_CUDA_TRY(cudaMemcpy(&bits, L->dev_status, 4, cudaMemcpyDeviceToHost));
    if (bits) ARISTOS_CUDA_TRY(cudaMemset(L->dev_status, 0, 4));
    if (bits & DEV_FAULT_TIMEOUT) { set_last_error("a bounded device-side wait expired"); return ARISTOS_ERR_DEVICE_TIMEOUT; }
    if (bits & DEV_FAULT_BOUNDS) { set_last_error("a routing index was out of range"); return ARISTOS_ERR_DEVICE_BOUNDS; }
    if (bits & DEV_FAULT_SCREEN) {
        set_last_error("the gate's tensor-core screen exceeded its error bound (affected tokens were re-evaluated "
                       "exactly; ARISTOS_GATE=exact selects the all-experts gate)");
        return ARISTOS_ERR_GATE_SCREEN;
    }
    if (bits & DEV_FAULT_NONFINITE) { set_last_error("a token's gate logits were NaN"); return ARISTOS_ERR_NONFINITE; }
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_set_profiling(aristos_moe_t* L, int enable) {
    if (!L) return ARISTOS_ERR_INVALID_ARG;
    if (enable && L->ev_prof.empty()) {
        L->ev_prof.assign(aristos_moe::PROF_SETS * aristos_moe::PROF_EVENTS, nullptr);
        for (cudaEvent_t& e : L->ev_prof) ARISTOS_CUDA_TRY(cudaEventCreate(&e));
    }
    L->profiling = enable != 0;
    L->prof_n = 0;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_stage_ms(aristos_moe_t* L, float out_ms[5]) {
    if (!L || !out_ms) return ARISTOS_ERR_INVALID_ARG;
    if (L->prof_n == 0) { set_last_error("stage_ms: no forward has run since profiling was switched on"); return ARISTOS_ERR_INVALID_ARG; }
    const int n = (int)std::min<int64_t>(L->prof_n, aristos_moe::PROF_SETS);
    double acc[5] = {0, 0, 0, 0, 0};
    for (int j = 0; j < n; ++j) {
        const int set = (int)((L->prof_n - 1 - j) % aristos_moe::PROF_SETS) * aristos_moe::PROF_EVENTS;
        ARISTOS_CUDA_TRY(cudaEventSynchronize(L->ev_prof[set + 4]));
        for (int i = 0; i < 5; ++i) {
            float ms = 0.0f;
            ARISTOS_CUDA_TRY(cudaEventElapsedTime(&ms, L->ev_prof[set + (i < 4 ? i : 0)], L->ev_prof[set + (i < 4 ? i + 1 : 4)]));
            acc[i] += ms;
        }
    }
    for (int i = 0; i < 5; ++i) out_ms[i] = (float)(acc[i] / n);
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_exchange_ms(aristos_moe_t* L, float* sent_ms) {
    if (!L || !sent_ms) return ARISTOS_ERR_INVALID_ARG;
    if (L->prof_n == 0) { set_last_error("exchange_ms: no forward has run since profiling was switched on"); return ARISTOS_ERR_INVALID_ARG; }
    *sent_ms = 0.0f;
    if (!(L->p2p && L->ep_direct) || L->fp8) return ARISTOS_OK;      // only the direct bf16 / fp16 / tf32 exchange marks it
    const int n = (int)std::min<int64_t>(L->prof_n, aristos_moe::PROF_SETS);
    double acc = 0;
    for (int j = 0; j < n; ++j) {
        const int set = (int)((L->prof_n - 1 - j) % aristos_moe::PROF_SETS) * aristos_moe::PROF_EVENTS;
        ARISTOS_CUDA_TRY(cudaEventSynchronize(L->ev_prof[set + 4]));
        ARISTOS_CUDA_TRY(cudaEventSynchronize(L->ev_prof[set + 5]));
        float ms = 0.0f;
        ARISTOS_CUDA_TRY(cudaEventElapsedTime(&ms, L->ev_prof[set + 2], L->ev_prof[set + 5]));
        acc += ms;
    }
    *sent_ms = (float)(acc / n);
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_exchange_profile(aristos_moe_t* L, float* ms4) {
    if (!L || !ms4) return ARISTOS_ERR_INVALID_ARG;
    if (L->prof_n == 0) { set_last_error("exchange_profile: no forward has run since profiling was switched on"); return ARISTOS_ERR_INVALID_ARG; }
    for (int i = 0; i < 4; ++i) ms4[i] = 0.0f;
    if (!(L->p2p && L->ep_direct) || L->fp8 || !L->prof_exchange) return ARISTOS_OK;
    const int n = (int)std::min<int64_t>(L->prof_n, aristos_moe::PROF_SETS);
    double acc[4] = {0, 0, 0, 0};
    for (int j = 0; j < n; ++j) {
        const int set = (int)((L->prof_n - 1 - j) % aristos_moe::PROF_SETS) * aristos_moe::PROF_EVENTS;
        ARISTOS_CUDA_TRY(cudaEventSynchronize(L->ev_prof[set + 4]));
        ARISTOS_CUDA_TRY(cudaEventSynchronize(L->ev_prof[set + 5]));
        // dispatch end -> rows sent | dispatch end -> counts arrived | counts arrived -> GEMMs done | -> returns arrived
        const int from[4] = {2, 2, 6, 7}, to[4] = {5, 6, 7, 3};
        for (int i = 0; i < 4; ++i) {
            float ms = 0.0f;
            ARISTOS_CUDA_TRY(cudaEventElapsedTime(&ms, L->ev_prof[set + from[i]], L->ev_prof[set + to[i]]));
            acc[i] += ms;
        }
    }
    for (int i = 0; i < 4; ++i) ms4[i] = (float)(acc[i] / n);
    return ARISTOS_OK;
}

size_t aristos_moe_training_bytes(const aristos_moe_t* L) { return (L && L->cfg.is_training) ? training_bytes(L) : 0; }

aristos_status_t aristos_moe_set_training_buffer(aristos_moe_t* L, void* device_buffer, size_t bytes) {
    if (!L) return ARISTOS_ERR_INVALID_ARG;
    if (!L->cfg.is_training) { set_last_error("set_training_buffer: the layer was created with is_training = 0"); return ARISTOS_ERR_CONFIG; }
    if (device_buffer && (bytes < training_bytes(L) || reinterpret_cast<uintptr_t>(device_buffer) % 256 != 0)) {
        set_last_error("set_training_buffer: %zu bytes given, %zu needed, 256-byte aligned", bytes, training_bytes(L));
        return ARISTOS_ERR_WORKSPACE;
    }
    L->train_buf = device_buffer;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_training_state(const aristos_moe_t* L, aristos_training_state_t* out) {
    if (!L || !out) return ARISTOS_ERR_INVALID_ARG;
    if (!L->cfg.is_training) { set_last_error("training_state: the layer was created with is_training = 0"); return ARISTOS_ERR_CONFIG; }
    if (!L->train_last.topk_idx) { set_last_error("training_state: no forward has run yet"); return ARISTOS_ERR_INVALID_ARG; }
    *out = L->train_last;
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_training_state_to_host(const aristos_moe_t* L, int32_t* topk_idx_host, float* topk_w_host,
                                                    int32_t* slot_of_host, float* load_balance_host) {
    aristos_training_state_t ts;
    ARISTOS_TRY(aristos_moe_training_state(L, &ts));
    if (L->world > 1 && L->ev_last_valid) ARISTOS_TRY(wait_event_bounded(const_cast<aristos_moe_t*>(L), L->ev_last));
    ARISTOS_CUDA_TRY(cudaDeviceSynchronize());
    const size_t sk = (size_t)ts.tokens * ts.top_k * 4;
    if (topk_idx_host) ARISTOS_CUDA_TRY(cudaMemcpy(topk_idx_host, ts.topk_idx, sk, cudaMemcpyDeviceToHost));
    if (topk_w_host) ARISTOS_CUDA_TRY(cudaMemcpy(topk_w_host, ts.topk_w, sk, cudaMemcpyDeviceToHost));
    if (slot_of_host) ARISTOS_CUDA_TRY(cudaMemcpy(slot_of_host, ts.slot_of, sk, cudaMemcpyDeviceToHost));
    if (load_balance_host)
        ARISTOS_CUDA_TRY(cudaMemcpy(load_balance_host, ts.load_balance, (size_t)(2 * ts.num_experts + 2) * 4, cudaMemcpyDeviceToHost));
    return ARISTOS_OK;
}

aristos_status_t aristos_moe_set_timeout_ms(aristos_moe_t* L, int timeout_ms) {
    if (!L || timeout_ms < 1) { set_last_error("set_timeout_ms: the limit must be at least 1 ms"); return ARISTOS_ERR_INVALID_ARG; }
    L->timeout_ms = timeout_ms;
    return ARISTOS_OK;
}

const char* aristos_moe_ep_transport(const aristos_moe_t* L) {
    if (!L || L->world == 1) return "none";
    return L->p2p ? "p2p" : "nccl";
}

int64_t aristos_moe_launch_count(const aristos_moe_t* L) { return L ? L->launches : 0; }

aristos_status_t aristos_moe_destroy(aristos_moe_t* L) {
    if (!L) return ARISTOS_OK;
    // a forward still waiting for a peer that will never come must not keep destroy from returning
    if (L->world > 1 && L->ev_last_valid && !L->failed) {
        const int keep = L->timeout_ms;
        L->timeout_ms = std::min(keep, 5000);
        wait_event_bounded(L, L->ev_last);
        L->timeout_ms = keep;
    }
    if (!(L->failed && !L->p2p)) cudaDeviceSynchronize();   // a stuck NCCL kernel cannot be waited for
    if (L->ev_last) cudaEventDestroy(L->ev_last);
    for (cudaEvent_t e : L->ev_in) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : L->ev_out) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : L->ev_prof) if (e) cudaEventDestroy(e);
    if (L->ev_dispatched) cudaEventDestroy(L->ev_dispatched);
    if (L->ev_returned) cudaEventDestroy(L->ev_returned);
    if (L->comm_stream) cudaStreamDestroy(L->comm_stream);
    for (auto& sl : L->slots) {
        if (sl.h2d_done) cudaEventDestroy(sl.h2d_done);
        if (sl.compute_done) cudaEventDestroy(sl.compute_done);
        if (sl.d2h_done) cudaEventDestroy(sl.d2h_done);
    }
    if (L->h2d_stream) cudaStreamDestroy(L->h2d_stream);
    if (L->d2h_stream) cudaStreamDestroy(L->d2h_stream);
    if (L->p2p) ep_p2p_destroy(L->p2p);
    if (L->comm) ep_comm_destroy(L->comm);
    if (L->ws && L->ws_owned) cudaFree(L->ws);
    delete L;
    return ARISTOS_OK;
}

}  // extern "C"
