// Helper for the column-sharded multi-GPU GEMM: after the all-gather of the per-rank output
// slabs, interleave them into the row-major result.  HBM-bound copy (read + write of C once).
#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace tbn_cuda {
namespace {

// One thread moves one float4 (or one float on the ragged path).
template <bool VEC>
__global__ void __launch_bounds__(256) gather_cols_permute_kernel(const float* __restrict__ slabs, int64_t G, int64_t M,
                                                                  int64_t Nc, float* __restrict__ c, int64_t ldc) {
    const int64_t per_row = VEC ? Nc / 4 : Nc;
    const int64_t total = G * M * per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t col = i % per_row;
        const int64_t gm = i / per_row;
        const int64_t m = gm % M, g = gm / M;
        if (VEC) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(slabs + (g * M + m) * Nc) + col);
            *(reinterpret_cast<float4*>(c + m * ldc + g * Nc) + col) = v;
        } else {
            c[m * ldc + g * Nc + col] = __ldg(slabs + (g * M + m) * Nc + col);
        }
    }
}

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" int32_t tbn_gather_cols_permute(const float* d_slabs, int64_t G, int64_t M, int64_t Nc, float* d_c,
                                           int64_t ldc, void* stream) {
    TBN_REQUIRE(G > 0 && M > 0 && Nc > 0, TBN_INVALID_SHAPE, "tbn_gather_cols_permute: dims must be positive");
    TBN_REQUIRE(d_slabs && d_c && ldc >= G * Nc, TBN_INVALID_ARGUMENT, "tbn_gather_cols_permute: bad arguments");
    const bool vec = Nc % 4 == 0 && ldc % 4 == 0 && reinterpret_cast<uintptr_t>(d_slabs) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(d_c) % 16 == 0;
    const int64_t total = G * M * (vec ? Nc / 4 : Nc);
    const int64_t cap = static_cast<int64_t>(sm_count() > 0 ? sm_count() : 148) * 16;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min((total + 255) / 256, cap)));
    if (vec) gather_cols_permute_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(d_slabs, G, M, Nc, d_c, ldc);
    else gather_cols_permute_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(d_slabs, G, M, Nc, d_c, ldc);
    return launched("gather_cols_permute_kernel");
}

// ---- sharing a device buffer between the processes of one box (one process per GPU) ---------------------
// The column-sharded GEMM writes its slab into every rank's result matrix; a rank makes its matrix reachable
// for the others by exporting an inter-process handle, the others open it and get a pointer in their own address
// space that tbn_gemm_fxb_multi accepts as a destination.  Thin wrappers of the CUDA IPC calls with the library's
// status convention.

extern "C" int32_t tbn_ipc_export(void* d_ptr, void* handle64) {
    TBN_REQUIRE(d_ptr && handle64, TBN_INVALID_ARGUMENT, "tbn_ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == TBN_IPC_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    TBN_CUDA_TRY(cudaIpcGetMemHandle(&h, d_ptr));
    std::memcpy(handle64, &h, sizeof h);
    return TBN_SUCCESS;
}

extern "C" int32_t tbn_ipc_open(const void* handle64, void** d_ptr) {
    TBN_REQUIRE(handle64 && d_ptr, TBN_INVALID_ARGUMENT, "tbn_ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof h);
    *d_ptr = nullptr;
    TBN_CUDA_TRY(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return TBN_SUCCESS;
}

extern "C" int32_t tbn_ipc_close(void* d_ptr) {
    if (d_ptr) TBN_CUDA_TRY(cudaIpcCloseMemHandle(d_ptr));
    return TBN_SUCCESS;
}
