// Shared declarations of the sm_100a kernels behind the C ABI in include/realq_b200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/realq_b200.h"

namespace rq {

// Device-side waits give up after this many SM clock cycles (about a second) and
// report RQ_ERR_TIMEOUT through the status word instead of spinning for ever.
constexpr long long kWaitCycles = 2000000000LL;

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? RQ_OK : RQ_ERR_CUDA;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Optional per-launch device timing (see rq_profile_enable); no-ops unless enabled.
namespace prof {
bool enabled();
void begin(int tag, cudaStream_t st, size_t* handle);
void end(size_t handle, cudaStream_t st);
struct Scope {
    size_t h;
    cudaStream_t st;
    Scope(int tag, cudaStream_t s) : st(s) { begin(tag, s, &h); }
    ~Scope() { end(h, st); }
};
}  // namespace prof

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, int64_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
    return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }

template <typename T>
__device__ __forceinline__ void store_from_float(T* p, int64_t i, float v);
template <>
__device__ __forceinline__ void store_from_float<float>(float* p, int64_t i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void store_from_float<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) {
    p[i] = __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ void store_from_float<__half>(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }

// clamp(rint(x / scale), lo, hi): true IEEE division and round-half-even, the arithmetic
// of torch.clamp(torch.round(x / scale), lo, hi).
__device__ __forceinline__ float quant_code(float x, float scale, float lo, float hi) {
    const float q = rintf(__fdiv_rn(x, scale));
    return q < lo ? lo : (q > hi ? hi : q);               // NaN propagates like torch.clamp
}

}  // namespace rq
