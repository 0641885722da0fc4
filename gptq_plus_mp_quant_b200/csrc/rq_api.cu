// Library-level entry points of the C ABI.
#include "rq_common.cuh"

extern "C" int rq_version(void) { return 100; }

extern "C" const char* rq_error_string(int code) {
    switch (code) {
        case RQ_OK: return "ok";
        case RQ_ERR_INVALID: return "invalid argument";
        case RQ_ERR_CUDA: return "CUDA runtime or driver call failed";
        case RQ_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case RQ_ERR_WORKSPACE: return "workspace too small";
        case RQ_ERR_UNSUPPORTED: return "configuration not supported by this build";
        case RQ_ERR_TOO_LARGE: return "problem exceeds the fixed 64 MiB scratch of the allocation-free entry point";
        default: return "unknown status";
    }
}

// ------------------------------------------------------------------------------------------
// Per-kernel device timing for benchmarks: when enabled, the launch sites of the dominant
// kernels bracket each launch with a pair of CUDA events on the launching stream.
// ------------------------------------------------------------------------------------------
#include <mutex>
#include <vector>

namespace rq {
namespace prof {
struct Span { cudaEvent_t a, b; int tag; };
static bool g_on = false;
static std::vector<Span> g_spans;
static std::mutex g_mu;

bool enabled() { return g_on; }

void begin(int tag, cudaStream_t st, size_t* handle) {
    *handle = (size_t)-1;
    if (!g_on) return;
    Span s;
    s.tag = tag;
    if (cudaEventCreate(&s.a) != cudaSuccess) return;
    if (cudaEventCreate(&s.b) != cudaSuccess) { cudaEventDestroy(s.a); return; }
    cudaEventRecord(s.a, st);
    std::lock_guard<std::mutex> lk(g_mu);
    g_spans.push_back(s);
    *handle = g_spans.size() - 1;
}

void end(size_t handle, cudaStream_t st) {
    if (handle == (size_t)-1) return;
    std::lock_guard<std::mutex> lk(g_mu);
    if (handle < g_spans.size()) cudaEventRecord(g_spans[handle].b, st);
}
}  // namespace prof
}  // namespace rq

extern "C" int rq_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(rq::prof::g_mu);
    for (auto& s : rq::prof::g_spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
    rq::prof::g_spans.clear();
    rq::prof::g_on = on != 0;
    return RQ_OK;
}

extern "C" int rq_profile_read(int tag, double* total_ms, long long* launches) {
    if (!total_ms || !launches) return RQ_ERR_INVALID;
    std::lock_guard<std::mutex> lk(rq::prof::g_mu);
    double tot = 0.0;
    long long n = 0;
    for (auto& s : rq::prof::g_spans) {
        if (s.tag != tag) continue;
        if (cudaEventSynchronize(s.b) != cudaSuccess) return RQ_ERR_CUDA;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, s.a, s.b) != cudaSuccess) return RQ_ERR_CUDA;
        tot += ms;
        ++n;
    }
    *total_ms = tot;
    *launches = n;
    return RQ_OK;
}
