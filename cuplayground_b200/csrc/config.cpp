// Run-time reader of aristos_config.json.
//
// The reference reads this file at configure time with CMake's string(JSON ...) and forwards the values as -D
// macros (CMakeLists.txt:167-216); the rules enforced here are those of aristos_config.schema.json:1-71 plus the
// extension keys documented in include/aristos_moe.h.
#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "common.cuh"

namespace aristos {
namespace {

// Minimal JSON reader: one top-level object whose known keys hold numbers (or true/false); any other value is
// skipped after being checked for well-formedness.
struct Parser {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p; }
    bool fail(const std::string& m) { if (err.empty()) err = m; return false; }
    bool expect(char c) {
        ws();
        if (p < end && *p == c) { ++p; return true; }
        return fail(std::string("expected '") + c + "'");
    }
    bool string(std::string& out) {
        ws();
        if (p >= end || *p != '"') return fail("expected string");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (p + 1 >= end) return fail("bad escape");
                out.push_back(p[1]);
                p += 2;
            } else {
                out.push_back(*p++);
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool number(double& v) {
        ws();
        if (p < end && !strncmp(p, "true", 4) && end - p >= 4) { v = 1; p += 4; return true; }
        if (p < end && !strncmp(p, "false", 5) && end - p >= 5) { v = 0; p += 5; return true; }
        char* q = nullptr;
        v = strtod(p, &q);
        if (q == p || q > end) return fail("expected number");
        p = q;
        return true;
    }
    bool skip_value(int depth = 0) {
        if (depth > 32) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        if (*p == '"') { std::string s; return string(s); }
        if (*p == '{' || *p == '[') {
            const char close = (*p == '{') ? '}' : ']';
            const bool obj = (*p == '{');
            ++p;
            ws();
            if (p < end && *p == close) { ++p; return true; }
            for (;;) {
                if (obj) { std::string k; if (!string(k) || !expect(':')) return false; }
                if (!skip_value(depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == close) { ++p; return true; }
                return fail("expected ',' or close");
            }
        }
        if (!strncmp(p, "null", 4) && end - p >= 4) { p += 4; return true; }
        double v;
        return number(v);
    }
};

bool is_integer(double v) { return std::floor(v) == v && std::fabs(v) < 2147483648.0; }

}  // namespace
}  // namespace aristos

using namespace aristos;

extern "C" {

aristos_status_t aristos_config_default(aristos_config_t* c) {
    if (!c) return ARISTOS_ERR_INVALID_ARG;
    memset(c, 0, sizeof(*c));
    // values shipped in aristos_config.json:2-12
    c->capacity_factor = 1.0;
    c->drop_tokens = 0;
    c->expert_top_k = 1;
    c->is_training = 0;
    c->hidden_act = ARISTOS_ACT_RELU;
    c->hidden_size = 1024;
    c->intermediate_size = 4096;
    c->micro_batch = 4;
    c->num_experts = 1;
    c->sequence_len = 2048;
    c->torch_dtype = ARISTOS_DTYPE_F32;
    c->tokens = 0;
    c->gate_fn = ARISTOS_GATE_SOFTMAX;
    c->renorm_topk = 0;
    c->gate_bias_zipf_s = 0.0;
    c->ep_world = 1;
    c->seed = 0;
    return ARISTOS_OK;
}

aristos_status_t aristos_config_parse(const char* text, aristos_config_t* out) {
    if (!text || !out) return ARISTOS_ERR_INVALID_ARG;
    aristos_config_t c;
    aristos_config_default(&c);
    Parser ps{text, text + strlen(text), {}};
    // keys the schema marks "required" (aristos_config.schema.json:59-70)
    static const char* required[] = {"hidden_act", "hidden_size", "intermediate_size", "expert_top_k",
                                     "capacity_factor", "drop_tokens", "num_experts", "sequence_len",
                                     "micro_batch", "torch_dtype"};
    bool seen[10] = {false};
    if (!ps.expect('{')) { set_last_error("config: %s", ps.err.c_str()); return ARISTOS_ERR_CONFIG; }
    ps.ws();
    bool first = true;
    while (ps.p < ps.end && *ps.p != '}') {
        if (!first && !ps.expect(',')) break;
        first = false;
        std::string key;
        if (!ps.string(key) || !ps.expect(':')) break;
        struct IntKey { const char* name; int* dst; };
        const IntKey ints[] = {{"drop_tokens", &c.drop_tokens}, {"expert_top_k", &c.expert_top_k},
                               {"is_training", &c.is_training}, {"hidden_act", &c.hidden_act},
                               {"hidden_size", &c.hidden_size}, {"intermediate_size", &c.intermediate_size},
                               {"micro_batch", &c.micro_batch}, {"num_experts", &c.num_experts},
                               {"sequence_len", &c.sequence_len}, {"torch_dtype", &c.torch_dtype},
                               {"tokens", &c.tokens}, {"gate_fn", &c.gate_fn}, {"renorm_topk", &c.renorm_topk},
                               {"ep_world", &c.ep_world}};
        bool known = false;
        for (const IntKey& ik : ints) {
            if (key == ik.name) {
                double v;
                if (!ps.number(v)) break;
                if (!is_integer(v)) { ps.fail("key '" + key + "' must be an integer"); break; }
                *ik.dst = (int)v;
                known = true;
                break;
            }
        }
        if (!ps.err.empty()) break;
        if (!known) {
            double v;
            if (key == "capacity_factor") { if (!ps.number(v)) break; c.capacity_factor = v; }
            else if (key == "gate_bias_zipf_s") { if (!ps.number(v)) break; c.gate_bias_zipf_s = v; }
            else if (key == "seed") { if (!ps.number(v)) break; c.seed = (uint64_t)v; }
            else if (!ps.skip_value()) break;
        }
        for (int i = 0; i < 10; ++i) if (key == required[i]) seen[i] = true;
        ps.ws();
    }
    if (ps.err.empty()) ps.expect('}');
    if (!ps.err.empty()) {
        set_last_error("config: %s (at offset %ld)", ps.err.c_str(), (long)(ps.p - text));
        return ARISTOS_ERR_CONFIG;
    }
    for (int i = 0; i < 10; ++i)
        if (!seen[i]) { set_last_error("config: required key '%s' is missing", required[i]); return ARISTOS_ERR_CONFIG; }
    aristos_status_t s = aristos_config_validate(&c);
    if (s != ARISTOS_OK) return s;
    *out = c;
    return ARISTOS_OK;
}

aristos_status_t aristos_config_load(const char* path, aristos_config_t* out) {
    if (!path || !out) return ARISTOS_ERR_INVALID_ARG;
    FILE* f = fopen(path, "rb");
    if (!f) { set_last_error("config: cannot open '%s'", path); return ARISTOS_ERR_IO; }
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
    return aristos_config_parse(text.c_str(), out);
}

#define CFG_REQUIRE(cond, ...)                                                  \
    do { if (!(cond)) { set_last_error("config: " __VA_ARGS__); return ARISTOS_ERR_CONFIG; } } while (0)

aristos_status_t aristos_config_validate(const aristos_config_t* c) {
    if (!c) return ARISTOS_ERR_INVALID_ARG;
    CFG_REQUIRE(c->capacity_factor > 0.0 && std::isfinite(c->capacity_factor), "capacity_factor must be > 0");
    CFG_REQUIRE(c->drop_tokens == 0 || c->drop_tokens == 1, "drop_tokens must be 0 or 1");
    CFG_REQUIRE(c->expert_top_k >= 1, "expert_top_k must be >= 1");
    CFG_REQUIRE(c->is_training == 0 || c->is_training == 1, "is_training must be 0 or 1");
    CFG_REQUIRE(c->hidden_act >= 0 && c->hidden_act <= 2, "hidden_act must be 0 (relu), 1 (gelu) or 2 (swiglu)");
    CFG_REQUIRE(c->hidden_size > 0 && c->hidden_size % 64 == 0, "hidden_size must be a positive multiple of 64");
    CFG_REQUIRE(c->intermediate_size > 0 && c->intermediate_size % 64 == 0,
                "intermediate_size must be a positive multiple of 64");
    CFG_REQUIRE(c->num_experts >= 1, "num_experts must be >= 1");
    CFG_REQUIRE(c->torch_dtype >= 0 && c->torch_dtype <= 4, "torch_dtype must be in 0..4");
    CFG_REQUIRE(c->tokens >= 0, "tokens must be >= 0");
    if (c->tokens == 0) {
        CFG_REQUIRE(c->micro_batch > 0 && c->micro_batch % 2 == 0, "micro_batch must be a positive multiple of 2");
        CFG_REQUIRE(c->sequence_len > 0 && c->sequence_len % 128 == 0,
                    "sequence_len must be a positive multiple of 128");
        CFG_REQUIRE((int64_t)c->micro_batch * c->sequence_len <= (1 << 24), "micro_batch*sequence_len too large");
    } else {
        CFG_REQUIRE(c->tokens <= (1 << 24), "tokens too large");
    }
    CFG_REQUIRE(c->gate_fn == 0 || c->gate_fn == 1, "gate_fn must be 0 (softmax) or 1 (sigmoid)");
    CFG_REQUIRE(c->renorm_topk == 0 || c->renorm_topk == 1, "renorm_topk must be 0 or 1");
    CFG_REQUIRE(c->gate_bias_zipf_s >= 0.0, "gate_bias_zipf_s must be >= 0");
    CFG_REQUIRE(c->ep_world >= 1, "ep_world must be >= 1");
    // constraints of the kernels of this build
    CFG_REQUIRE(c->expert_top_k <= c->num_experts, "expert_top_k must not exceed num_experts");
    CFG_REQUIRE(c->expert_top_k <= 16, "expert_top_k must be <= 16");
    CFG_REQUIRE(c->num_experts <= 1024, "num_experts must be <= 1024");
    CFG_REQUIRE(c->num_experts % c->ep_world == 0, "num_experts must be divisible by ep_world");
    return ARISTOS_OK;
}

int aristos_config_tokens(const aristos_config_t* c) {
    if (!c) return 0;
    return c->tokens > 0 ? c->tokens : c->micro_batch * c->sequence_len;
}

int aristos_config_capacity(const aristos_config_t* c) {
    if (!c) return 0;
    const int S = aristos_config_tokens(c);
    if (!c->drop_tokens) return S;
    double cap = std::ceil(c->capacity_factor * (double)S * (double)c->expert_top_k / (double)c->num_experts - 1e-9);
    if (cap < 1.0) cap = 1.0;
    if (cap > (double)S) cap = (double)S;
    return (int)cap;
}

aristos_status_t aristos_zipf_bias_host(float* bias, int E, double s) {
    if (!bias || E < 1) return ARISTOS_ERR_INVALID_ARG;
    for (int e = 0; e < E; ++e) bias[e] = (float)(-s * std::log((double)(e + 1)));
    return ARISTOS_OK;
}

}  // extern "C"
