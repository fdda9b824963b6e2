// Host-only entry point to the seeded model writer, for the benchmark's CPU arm (TEST INFRASTRUCTURE, like the
// rest of this folder): the arm that times the CPU restatement needs the same synthetic GGUF the GPU arm runs
// and must not load the GPU library to get it. The writer itself is retrograd_b200/csrc/synth.cpp, compiled
// into this small library as it stands (it depends on nothing but the C++ standard library).
#include <cstdint>
#include <exception>
#include <string>

namespace rb200 {
uint64_t synth_gguf(const char * path, const char * spec_text);
}

namespace {
thread_local std::string g_error;
}

extern "C" {

const char * ora_modelgen_last_error(void) { return g_error.c_str(); }

// spec: whitespace-separated key=value pairs (the keys of retro_b200_synth_gguf). 0 on success.
int ora_synth_gguf(const char * path, const char * spec, uint64_t * out_bytes) {
    try {
        const uint64_t n = rb200::synth_gguf(path, spec);
        if (out_bytes) *out_bytes = n;
        return 0;
    } catch (const std::exception & err) {
        g_error = err.what();
        return -1;
    }
}

} // extern "C"
