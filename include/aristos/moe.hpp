// C++ host API over the C ABI of aristos_moe.h: RAII handles, exceptions instead of status codes.
//
// This is the callable form of what the reference's harnesses do by hand (load the configuration, allocate, launch,
// synchronise, free - mma.cuh:371-443, auditorium/overlap.cuh:159-242). Header-only; link libaristos_moe.so.
#pragma once

#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>

#include "../aristos_moe.h"

namespace aristos {

class Error : public std::runtime_error {
public:
    Error(aristos_status_t s, const std::string& what) : std::runtime_error(what), status_(s) {}
    aristos_status_t status() const noexcept { return status_; }

private:
    aristos_status_t status_;
};

inline void check(aristos_status_t s) {
    if (s != ARISTOS_OK) throw Error(s, std::string(aristos_status_str(s)) + ": " + aristos_last_error());
}

// aristos_config.json (reference keys + extension keys), validated on construction.
class Config {
public:
    Config() { check(aristos_config_default(&c_)); }
    static Config load(const std::string& json_path) {
        Config c;
        check(aristos_config_load(json_path.c_str(), &c.c_));
        return c;
    }
    static Config parse(const std::string& json_text) {
        Config c;
        check(aristos_config_parse(json_text.c_str(), &c.c_));
        return c;
    }
    void validate() const { check(aristos_config_validate(&c_)); }
    int tokens() const { return aristos_config_tokens(&c_); }
    int capacity() const { return aristos_config_capacity(&c_); }
    aristos_config_t& raw() noexcept { return c_; }
    const aristos_config_t& raw() const noexcept { return c_; }

private:
    aristos_config_t c_;
};

// One MoE layer on the CUDA device that is current at construction.
class MoeLayer {
public:
    // nccl_unique_id: 128 bytes from unique_id() on rank 0, shared with every rank; nullptr when world == 1.
    explicit MoeLayer(const Config& cfg, int rank = 0, int world = 1, const void* nccl_unique_id = nullptr) {
        check(aristos_moe_create(&cfg.raw(), rank, world, nccl_unique_id, &h_));
    }
    ~MoeLayer() { aristos_moe_destroy(h_); }
    MoeLayer(const MoeLayer&) = delete;
    MoeLayer& operator=(const MoeLayer&) = delete;
    MoeLayer(MoeLayer&& o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
    MoeLayer& operator=(MoeLayer&& o) noexcept {
        if (this != &o) { aristos_moe_destroy(h_); h_ = std::exchange(o.h_, nullptr); }
        return *this;
    }

    static void unique_id(void* out_128_bytes) { check(aristos_nccl_unique_id(out_128_bytes)); }

    size_t workspace_bytes() const { return aristos_moe_workspace_bytes(h_); }
    void set_workspace(void* device_ptr, size_t bytes) { check(aristos_moe_set_workspace(h_, device_ptr, bytes)); }

    // Device tensors: x (S,H), w_gate (E,H), w1/w3 (E_local,I,H), w2 (E_local,H,I), out (S,H). Asynchronous on stream.
    void forward(const void* x, const void* w_gate, const void* w1, const void* w3, const void* w2, void* out,
                 void* stream = nullptr, const float* gate_bias = nullptr) {
        check(aristos_moe_forward(h_, x, w_gate, gate_bias, w1, w3, w2, nullptr, out, stream));
    }
    // Host activations in, host result out (weights stay on the device); returns when out_host is complete.
    void forward_host(const void* x_host, const void* w_gate, const void* w1, const void* w3, const void* w2,
                      void* out_host, void* stream = nullptr, const float* gate_bias = nullptr) {
        check(aristos_moe_forward_host(h_, x_host, w_gate, gate_bias, w1, w3, w2, nullptr, out_host, stream));
    }
    aristos_routing_t routing() const {
        aristos_routing_t r;
        check(aristos_moe_routing(h_, &r));
        return r;
    }
    // Synchronises and throws if a kernel reported a device-side fault (expired wait, bad routing index).
    void status() { check(aristos_moe_status(h_)); }
    void set_profiling(bool on) { check(aristos_moe_set_profiling(h_, on ? 1 : 0)); }
    struct StageMs { float gate, dispatch, ffn, combine, total; };
    StageMs stage_ms() {
        float ms[5];
        check(aristos_moe_stage_ms(h_, ms));
        return StageMs{ms[0], ms[1], ms[2], ms[3], ms[4]};
    }
    // Expert-parallel peer-memory layers: the expert-FFN stage split at its cross-rank waits (milliseconds).
    struct ExchangeMs { float rows_sent, counts_arrived, gemms, returns_arrived; };
    ExchangeMs exchange_profile() {
        float ms[4];
        check(aristos_moe_exchange_profile(h_, ms));
        return ExchangeMs{ms[0], ms[1], ms[2], ms[3]};
    }
    // Expert-parallel layers: wall-clock limit of status() / destruction when a peer stops taking part.
    void set_timeout_ms(int ms) { check(aristos_moe_set_timeout_ms(h_, ms)); }
    // is_training = 1: what the last forward saved (device pointers), and where the next forwards save.
    aristos_training_state_t training_state() const {
        aristos_training_state_t t;
        check(aristos_moe_training_state(h_, &t));
        return t;
    }
    size_t training_bytes() const { return aristos_moe_training_bytes(h_); }
    void set_training_buffer(void* device_ptr, size_t bytes) { check(aristos_moe_set_training_buffer(h_, device_ptr, bytes)); }
    const char* ep_transport() const { return aristos_moe_ep_transport(h_); }
    long long launch_count() const { return aristos_moe_launch_count(h_); }
    aristos_moe_t* raw() noexcept { return h_; }

private:
    aristos_moe_t* h_ = nullptr;
};

}  // namespace aristos
