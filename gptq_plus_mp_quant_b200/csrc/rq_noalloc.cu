// Hessian accumulation for callers that cannot allocate device memory.
//
// Some hosts of this library must not call cudaMalloc (or any allocating routine) on the path
// that feeds calibration batches: a forward hook that runs while a memory pool is frozen, a
// process whose device-memory budget is owned by another component, a caller that has no
// torch allocator to borrow scratch from.  rq_hessian_accum needs scratch for the bf16 operand
// planes it packs; here that scratch is a fixed array that lives in the library's device image,
// so the call needs nothing beyond its inputs and outputs.
#include <mutex>

#include "rq_common.cuh"

// 64 MiB per GPU that loads the library, held until the process exits.  The alignment is the one
// rq_hessian_accum demands of any workspace it is given (1024 bytes: the swizzled TMA tiles of the planes).
#define RQ_NOALLOC_SCRATCH_BYTES (64u * 1024u * 1024u)
static __device__ __align__(1024) unsigned char g_noalloc_scratch[RQ_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mu;

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address: the
// address on the CURRENT device has to be asked for, once per device.
int scratch_on_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RQ_ERR_CUDA;
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return RQ_ERR_CUDA;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return RQ_OK;
}
}  // namespace

extern "C" size_t rq_hessian_noalloc_scratch_bytes(void) { return RQ_NOALLOC_SCRATCH_BYTES; }

extern "C" int rq_hessian_accum_noalloc(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H,
                                        float* act_sq, int64_t N, int C, int G, float alpha, float beta, int* status,
                                        void* stream) {
    if (C <= 0 || G <= 0) return RQ_ERR_INVALID;
    // the smallest unit of work is a 64-token chunk; if even that does not fit, the problem is too wide
    if (rq_hessian_workspace_bytes(64, C, G, sal != nullptr) > (size_t)RQ_NOALLOC_SCRATCH_BYTES) return RQ_ERR_TOO_LARGE;
    void* scratch = nullptr;
    const int rc = scratch_on_current_device(&scratch);
    if (rc != RQ_OK) return rc;
    // rq_hessian_accum sizes its token chunks to the scratch it is given and writes every byte of the
    // planes it reads, so nothing in the array has to be cleared between calls.
    return rq_hessian_accum(x, x_dtype, ldx, sal, H, act_sq, N, C, G, alpha, beta, scratch,
                            (size_t)RQ_NOALLOC_SCRATCH_BYTES, status, 0, stream);
}
