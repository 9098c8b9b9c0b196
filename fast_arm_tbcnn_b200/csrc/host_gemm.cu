// Float x binary GEMM on HOST buffers: the activations arrive in host memory and the result is wanted
// in host memory, as with the reference's operators (tbn::Tensor is a host buffer there).  The rows of A
// are cut into chunks; chunk i+1 is uploaded and chunk i-1 is downloaded while chunk i is multiplied,
// on three internal streams with double-buffered device staging, so a step costs about
// max(upload, compute, download) instead of their sum.  The packed weights stay resident on the device.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace tbn_cuda {
namespace {

struct Pipeline {
    bool ready = false;
    cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
    cudaEvent_t a_ready[2] = {nullptr, nullptr}, c_done[2] = {nullptr, nullptr}, d2h_done[2] = {nullptr, nullptr};
    cudaEvent_t begin = nullptr, end_compute = nullptr;
    // Held while one call enqueues its work: the streams and events above are shared by every call on the device,
    // so two host threads (or two caller streams) must not interleave their records and waits.
    std::mutex enqueue;
};
constexpr int kMaxDev = 64;
Pipeline g_pipe[kMaxDev];
std::mutex g_pipe_mutex;

int32_t get_pipeline(Pipeline** out) {
    int dev = -1;
    TBN_CUDA_TRY(cudaGetDevice(&dev));
    TBN_REQUIRE(dev >= 0 && dev < kMaxDev, TBN_RUNTIME_ERROR, "device index out of range");
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    Pipeline& p = g_pipe[dev];
    if (!p.ready) {
        TBN_CUDA_TRY(cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking));
        TBN_CUDA_TRY(cudaStreamCreateWithFlags(&p.compute, cudaStreamNonBlocking));
        TBN_CUDA_TRY(cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            TBN_CUDA_TRY(cudaEventCreateWithFlags(&p.a_ready[i], cudaEventDisableTiming));
            TBN_CUDA_TRY(cudaEventCreateWithFlags(&p.c_done[i], cudaEventDisableTiming));
            TBN_CUDA_TRY(cudaEventCreateWithFlags(&p.d2h_done[i], cudaEventDisableTiming));
        }
        TBN_CUDA_TRY(cudaEventCreateWithFlags(&p.begin, cudaEventDisableTiming));
        TBN_CUDA_TRY(cudaEventCreateWithFlags(&p.end_compute, cudaEventDisableTiming));
        p.ready = true;
    }
    *out = &p;
    return TBN_SUCCESS;
}

// Rows per chunk: about sixteen chunks (the first upload and the last download are not overlapped, so shorter
// chunks shorten the call as long as a chunk still fills the GPU for several waves), whole 128-row tiles.
int64_t chunk_rows(int64_t M) {
    const int64_t parts = M >= 8192 ? 16 : 8;  // measured at 16384^3: 8 -> 25.1 ms, 16 -> 23.9 ms, 32 -> 26 ms
    const int64_t target = (M + parts - 1) / parts;
    return std::min<int64_t>(round_up(std::max<int64_t>(target, 128), 128), round_up(M, 128));
}

struct Layout {
    int64_t rows;
    size_t a_bytes, c_bytes, gemm_bytes, total;
};

Layout layout_for(int64_t M, int64_t K, int64_t N, int32_t mode) {
    Layout l;
    l.rows = chunk_rows(M);
    l.a_bytes = static_cast<size_t>(round_up(l.rows * K * 4, 256));
    l.c_bytes = static_cast<size_t>(round_up(l.rows * N * 4, 256));
    l.gemm_bytes = static_cast<size_t>(round_up(static_cast<int64_t>(tbn_gemm_workspace_bytes(l.rows, K, mode)), 256));
    l.total = 2 * l.a_bytes + 2 * l.c_bytes + l.gemm_bytes;
    return l;
}

}  // namespace
}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

size_t tbn_gemm_fxb_host_workspace_bytes(int64_t M, int64_t K, int64_t N, int32_t mode) {
    if (M <= 0 || K <= 0 || N <= 0) return 0;
    return layout_for(M, K, N, mode).total;
}

int32_t tbn_gemm_fxb_host(const float* h_a, int64_t M, int64_t K, int64_t lda, const uint32_t* d_neg,
                          const uint32_t* d_pos, int64_t N, const float* d_alpha, float scale, const float* d_bias,
                          float* h_c, int64_t ldc, int32_t mode, uint32_t epilogue, void* d_workspace,
                          size_t workspace_bytes, void* stream) {
    TBN_REQUIRE(M > 0 && N > 0 && K > 0, TBN_INVALID_SHAPE, "tbn_gemm_fxb_host: M, N and K must be positive");
    TBN_REQUIRE(h_a && h_c && d_neg, TBN_INVALID_ARGUMENT, "tbn_gemm_fxb_host: null pointer");
    TBN_REQUIRE(lda >= K && ldc >= N, TBN_INVALID_ARGUMENT, "tbn_gemm_fxb_host: leading dimension smaller than the row length");
    if (mode == TBN_MODE_AUTO) mode = TBN_MODE_TC_BF16X2;
    const Layout l = layout_for(M, K, N, mode);
    TBN_REQUIRE(d_workspace && workspace_bytes >= l.total, TBN_INVALID_ARGUMENT,
                "tbn_gemm_fxb_host: workspace too small (see tbn_gemm_fxb_host_workspace_bytes)");
    TBN_REQUIRE(reinterpret_cast<uintptr_t>(d_workspace) % 256 == 0, TBN_INVALID_ARGUMENT,
                "tbn_gemm_fxb_host: workspace must be 256-byte aligned");
    Pipeline* p = nullptr;
    int32_t rc = get_pipeline(&p);
    if (rc) return rc;
    std::lock_guard<std::mutex> enqueue_lock(p->enqueue);
    uint8_t* ws = static_cast<uint8_t*>(d_workspace);
    float* a_slot[2] = {reinterpret_cast<float*>(ws), reinterpret_cast<float*>(ws + l.a_bytes)};
    float* c_slot[2] = {reinterpret_cast<float*>(ws + 2 * l.a_bytes), reinterpret_cast<float*>(ws + 2 * l.a_bytes + l.c_bytes)};
    void* gemm_ws = ws + 2 * l.a_bytes + 2 * l.c_bytes;

    cudaStream_t user = as_stream(stream);
    TBN_CUDA_TRY(cudaEventRecord(p->begin, user));
    TBN_CUDA_TRY(cudaStreamWaitEvent(p->h2d, p->begin, 0));
    TBN_CUDA_TRY(cudaStreamWaitEvent(p->compute, p->begin, 0));
    TBN_CUDA_TRY(cudaStreamWaitEvent(p->d2h, p->begin, 0));
    const int64_t chunks = (M + l.rows - 1) / l.rows;
    for (int64_t i = 0; i < chunks; ++i) {
        const int s = static_cast<int>(i & 1);
        const int64_t m0 = i * l.rows, rows = std::min(l.rows, M - m0);
        // upload: the slot is free once the GEMM of chunk i-2 has consumed it
        if (i >= 2) TBN_CUDA_TRY(cudaStreamWaitEvent(p->h2d, p->c_done[s], 0));
        TBN_CUDA_TRY(cudaMemcpy2DAsync(a_slot[s], static_cast<size_t>(K) * 4, h_a + m0 * lda, static_cast<size_t>(lda) * 4,
                                       static_cast<size_t>(K) * 4, static_cast<size_t>(rows), cudaMemcpyHostToDevice, p->h2d));
        TBN_CUDA_TRY(cudaEventRecord(p->a_ready[s], p->h2d));
        // compute: needs the upload, and the result slot must have been drained by the download of chunk i-2
        TBN_CUDA_TRY(cudaStreamWaitEvent(p->compute, p->a_ready[s], 0));
        if (i >= 2) TBN_CUDA_TRY(cudaStreamWaitEvent(p->compute, p->d2h_done[s], 0));
        rc = tbn_gemm_fxb(a_slot[s], rows, K, K, d_neg, d_pos, N, d_alpha, scale, d_bias, c_slot[s], N, mode, epilogue, gemm_ws,
                          l.gemm_bytes, p->compute);
        if (rc) return rc;
        TBN_CUDA_TRY(cudaEventRecord(p->c_done[s], p->compute));
        // download
        TBN_CUDA_TRY(cudaStreamWaitEvent(p->d2h, p->c_done[s], 0));
        TBN_CUDA_TRY(cudaMemcpy2DAsync(h_c + m0 * ldc, static_cast<size_t>(ldc) * 4, c_slot[s], static_cast<size_t>(N) * 4,
                                       static_cast<size_t>(N) * 4, static_cast<size_t>(rows), cudaMemcpyDeviceToHost, p->d2h));
        TBN_CUDA_TRY(cudaEventRecord(p->d2h_done[s], p->d2h));
    }
    // The caller's stream continues only after the last download (both slots) has finished.
    TBN_CUDA_TRY(cudaStreamWaitEvent(user, p->d2h_done[0], 0));
    if (chunks > 1) TBN_CUDA_TRY(cudaStreamWaitEvent(user, p->d2h_done[1], 0));
    TBN_CUDA_TRY(cudaEventRecord(p->end_compute, p->h2d));
    TBN_CUDA_TRY(cudaStreamWaitEvent(user, p->end_compute, 0));
    return TBN_SUCCESS;
}

}  // extern "C"
