"""The C++ RAII header (include/aristos/moe.hpp) compiles with a plain C++17 compiler against the C ABI and its
host-only parts (configuration, error reporting) behave like the C entry points."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <aristos/moe.hpp>
#include <cstdio>
int main() {
    auto cfg = aristos::Config::parse(R"({"capacity_factor": 1.25, "drop_tokens": 1, "expert_top_k": 2, "hidden_act": 2,
        "hidden_size": 4096, "intermediate_size": 14336, "micro_batch": 4, "num_experts": 8, "sequence_len": 2048,
        "torch_dtype": 2, "tokens": 16384})");
    if (cfg.tokens() != 16384 || cfg.capacity() != 5120) return 2;
    try {
        aristos::Config::parse("{\"hidden_size\": 100}");
        return 3;
    } catch (const aristos::Error& e) {
        if (e.status() != ARISTOS_ERR_CONFIG) return 4;
    }
    try {
        aristos::MoeLayer layer(cfg);          // no CUDA device in the CPU test environment -> a CUDA error, not a crash
        std::printf("layer created (a GPU is present)\n");
    } catch (const aristos::Error& e) {
        if (e.status() != ARISTOS_ERR_CUDA) return 5;
        std::printf("no device: %s\n", e.what());
    }
    std::printf("ok\n");
    return 0;
}
'''


def test_cpp_header_compiles_and_runs(tmp_path):
    from cuplayground_b200 import build
    lib = build.build_library()
    src = tmp_path / "use_hpp.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "use_hpp"
    libdir = os.path.dirname(lib)
    subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                           str(src), "-o", str(exe), "-L", libdir, "-laristos_moe", f"-Wl,-rpath,{libdir}"])
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "ok" in r.stdout
