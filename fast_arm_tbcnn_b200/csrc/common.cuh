// Shared host/device helpers of the CUDA library: status + error message plumbing,
// launch bookkeeping, the epilogue every GEMM-shaped kernel applies, small PTX wrappers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/tbn_cuda.h"

namespace tbn_cuda {

// ---- host side -------------------------------------------------------------------

// Records `msg` as the calling thread's last error and returns `code`.
int32_t fail(int32_t code, const std::string& msg);
// Converts a CUDA runtime error into a status (OOM -> TBN_OUT_OF_MEMORY).
int32_t cuda_fail(cudaError_t err, const char* what);
// Counts one kernel launch and checks the launch itself.
int32_t launched(const char* kernel_name);
// Device pointer (in mapped pinned host memory) where kernels record a device-side
// error code; 0 = no error.  Valid after tbn_cuda_init on the current device.
int* device_error_word();
int sm_count();
// Benchmark instrumentation (tbn_cuda_profile_enable): records an event on `st` that opens
// (begin) or closes (end) the timing bracket of one kernel of the given kind.  No-ops while
// profiling is disabled.
enum ProfileKind : int { kProfGemm = 0, kProfSplit = 1 };
void profile_begin(ProfileKind kind, cudaStream_t st);
void profile_end(ProfileKind kind, cudaStream_t st);

#define TBN_CUDA_TRY(expr)                                         \
    do {                                                           \
        cudaError_t _e = (expr);                                   \
        if (_e != cudaSuccess) return ::tbn_cuda::cuda_fail(_e, #expr); \
    } while (0)

#define TBN_REQUIRE(cond, code, msg)                        \
    do {                                                    \
        if (!(cond)) return ::tbn_cuda::fail((code), (msg)); \
    } while (0)

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Device-side error codes written to device_error_word().
enum DeviceError : int {
    kErrNone = 0,
    kErrWaitEmpty = 1,      // producer / transform waited for a free smem stage
    kErrWaitFullA = 2,      // MMA waited for the TMA-loaded activation tile
    kErrWaitFullB = 3,      // MMA waited for the unpacked weight tile
    kErrWaitTmemFull = 4,   // epilogue waited for the accumulator
    kErrWaitTmemEmpty = 5,  // MMA waited for the epilogue to drain the accumulator
    kErrPackWaitFull = 6,   // weight pack: consumers waited for a TMA tile
    kErrPackWaitEmpty = 7,  // weight pack: the producer waited for a free stage
    kErrSelfTest = 8,       // tbn_cuda_selftest_wait_timeout: the wait that nothing completes
};

// ---- epilogue ----------------------------------------------------------------------

struct Epilogue {
    const float* alpha;     // [N] or nullptr
    const float* bias;      // [N] or nullptr
    const float* residual;  // same layout as the output, read when TBN_EPI_ADD_RESIDUAL is set
    float scale;
    uint32_t flags;
};

// Separate multiply and add (no FMA contraction) so that the integer-exact paths are
// bit-equal to the reference's `float(acc) * scale`, `+= bias`, `*= alpha` loops.
__device__ __forceinline__ float apply_epilogue(float acc, float alpha, float bias, float scale,
                                                uint32_t flags, float residual) {
    float v;
    if (flags & TBN_EPI_BIAS_BEFORE_ALPHA) {
        v = __fmul_rn(acc, scale);
        v = __fadd_rn(v, bias);
        v = __fmul_rn(v, alpha);
    } else {
        v = __fmul_rn(acc, alpha);
        v = __fmul_rn(v, scale);
        v = __fadd_rn(v, bias);
    }
    if (flags & TBN_EPI_ADD_RESIDUAL) v = __fadd_rn(v, residual);
    if (flags & TBN_EPI_RELU) v = fmaxf(v, 0.0f);
    return v;
}

}  // namespace tbn_cuda
