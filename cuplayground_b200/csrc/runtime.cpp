// Status strings, per-thread error text and small device queries of libaristos_moe.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace aristos {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

aristos_status_t cuda_fail(cudaError_t e, const char* what) {
    set_last_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return ARISTOS_ERR_CUDA;
}

int device_sm_count() {
    static thread_local int cached_dev = -1, cached_sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev != cached_dev) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached_dev = dev;
        cached_sms = sms;
    }
    return cached_sms;
}

int64_t& launch_counter() {
    static thread_local int64_t n = 0;
    return n;
}

}  // namespace aristos

extern "C" {

const char* aristos_status_str(aristos_status_t s) {
    switch (s) {
        case ARISTOS_OK: return "ok";
        case ARISTOS_ERR_INVALID_ARG: return "invalid argument";
        case ARISTOS_ERR_CONFIG: return "invalid configuration";
        case ARISTOS_ERR_IO: return "i/o error";
        case ARISTOS_ERR_CUDA: return "CUDA error";
        case ARISTOS_ERR_NCCL: return "NCCL error";
        case ARISTOS_ERR_UNSUPPORTED: return "unsupported";
        case ARISTOS_ERR_WORKSPACE: return "workspace too small";
        case ARISTOS_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case ARISTOS_ERR_DEVICE_BOUNDS: return "device-side index out of range";
        case ARISTOS_ERR_NOMEM: return "out of memory";
        case ARISTOS_ERR_GATE_SCREEN: return "gate screen error bound exceeded";
        case ARISTOS_ERR_NONFINITE: return "non-finite gate logits";
    }
    return "unknown status";
}

const char* aristos_last_error(void) { return aristos::g_last_error; }

int aristos_version(void) { return 100; }

}  // extern "C"
