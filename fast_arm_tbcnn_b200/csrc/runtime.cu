// Runtime part of the C ABI: device selection, device-resident tensor storage, copies,
// error plumbing.  Stands in for the host allocation inside tbn::Tensor
// (tbn/runtime/tensor.hpp:23-35) and for the exception messages of tbn/utils/errors.hpp.
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace tbn_cuda {

namespace {

thread_local std::string g_last_error;
std::atomic<int64_t> g_launches{0};

constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    int sms = 0;
    int* err_host = nullptr;  // mapped pinned host memory
    int* err_dev = nullptr;   // device alias of err_host
};
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mutex;

DeviceState* current_state() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    return g_dev[dev].ready ? &g_dev[dev] : nullptr;
}

}  // namespace

int32_t fail(int32_t code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int32_t cuda_fail(cudaError_t err, const char* what) {
    // Clear the sticky-less error so that the next call starts clean.
    cudaGetLastError();
    const int32_t code = (err == cudaErrorMemoryAllocation) ? TBN_OUT_OF_MEMORY : TBN_CUDA_ERROR;
    return fail(code, std::string(what) + ": " + cudaGetErrorString(err));
}

int32_t launched(const char* kernel_name) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, kernel_name);
    return TBN_SUCCESS;
}

int* device_error_word() {
    DeviceState* s = current_state();
    return s ? s->err_dev : nullptr;
}

int sm_count() {
    DeviceState* s = current_state();
    return s ? s->sms : 0;
}

namespace {
std::atomic<bool> g_profile{false};
struct ProfileSpan {
    cudaEvent_t start, stop;
    int kind;
};
std::mutex g_prof_mutex;
std::vector<ProfileSpan> g_spans;
cudaEvent_t g_open[2] = {nullptr, nullptr};
}  // namespace

void profile_begin(ProfileKind kind, cudaStream_t st) {
    if (!g_profile.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    cudaEvent_t ev;
    if (cudaEventCreate(&ev) != cudaSuccess) return;
    cudaEventRecord(ev, st);
    g_open[kind] = ev;
}

void profile_end(ProfileKind kind, cudaStream_t st) {
    if (!g_profile.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (!g_open[kind]) return;
    cudaEvent_t ev;
    if (cudaEventCreate(&ev) != cudaSuccess) return;
    cudaEventRecord(ev, st);
    g_spans.push_back({g_open[kind], ev, static_cast<int>(kind)});
    g_open[kind] = nullptr;
}

namespace {
// One thread waits on a barrier that nothing ever completes: the wait must run out by itself.
__global__ void wait_selftest_kernel(int* err_word) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        const uint32_t b = ptx::smem_u32(&bar);
        ptx::mbar_init(b, 1);
        ptx::fence_barrier_init();
        ptx::mbar_wait(b, 0, err_word, kErrSelfTest);
    }
}
}  // namespace

}  // namespace tbn_cuda

using namespace tbn_cuda;

extern "C" {

int32_t tbn_cuda_init(int32_t device) {
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(TBN_DEVICE_NOT_SUPPORTED,
                    "no CUDA device available; this library has no CPU fallback");
    }
    TBN_REQUIRE(device >= 0 && device < count && device < kMaxDevices, TBN_INVALID_ARGUMENT,
                "tbn_cuda_init: device index out of range");
    TBN_CUDA_TRY(cudaSetDevice(device));
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState& s = g_dev[device];
    if (s.ready) return TBN_SUCCESS;
    cudaDeviceProp prop;
    TBN_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        return fail(TBN_DEVICE_NOT_SUPPORTED,
                    std::string("device '") + prop.name + "' is compute capability " +
                        std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                        "; the kernels are built for sm_100a only");
    }
    s.sms = prop.multiProcessorCount;
    TBN_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&s.err_host), 64, cudaHostAllocMapped));
    std::memset(s.err_host, 0, 64);
    *reinterpret_cast<volatile uint64_t*>(s.err_host + ptx::kWaitLimitWordOffset) = ptx::kDefaultWaitLimitNs;
    TBN_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.err_dev), s.err_host, 0));
    s.ready = true;
    return TBN_SUCCESS;
}

int32_t tbn_cuda_last_error(char* buf, size_t buf_bytes) {
    if (buf && buf_bytes) {
        std::strncpy(buf, g_last_error.c_str(), buf_bytes - 1);
        buf[buf_bytes - 1] = '\0';
    }
    return static_cast<int32_t>(g_last_error.size());
}

int32_t tbn_cuda_malloc(void** d_ptr, size_t bytes) {
    TBN_REQUIRE(d_ptr != nullptr, TBN_INVALID_ARGUMENT, "tbn_cuda_malloc: null out pointer");
    *d_ptr = nullptr;
    if (bytes == 0) return TBN_SUCCESS;
    TBN_CUDA_TRY(cudaMalloc(d_ptr, bytes));
    // tbn::Tensor zero-fills on construction (tensor.hpp:27).
    TBN_CUDA_TRY(cudaMemset(*d_ptr, 0, bytes));
    return TBN_SUCCESS;
}

int32_t tbn_cuda_free(void* d_ptr) {
    if (d_ptr) TBN_CUDA_TRY(cudaFree(d_ptr));
    return TBN_SUCCESS;
}

int32_t tbn_cuda_memset(void* d_ptr, int32_t value, size_t bytes, void* stream) {
    if (bytes == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_ptr != nullptr, TBN_INVALID_ARGUMENT, "tbn_cuda_memset: null pointer");
    TBN_CUDA_TRY(cudaMemsetAsync(d_ptr, value, bytes, as_stream(stream)));
    return TBN_SUCCESS;
}

int32_t tbn_cuda_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream) {
    if (bytes == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_dst && h_src, TBN_INVALID_ARGUMENT, "tbn_cuda_h2d: null pointer");
    TBN_CUDA_TRY(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return TBN_SUCCESS;
}

int32_t tbn_cuda_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream) {
    if (bytes == 0) return TBN_SUCCESS;
    TBN_REQUIRE(h_dst && d_src, TBN_INVALID_ARGUMENT, "tbn_cuda_d2h: null pointer");
    TBN_CUDA_TRY(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return TBN_SUCCESS;
}

int32_t tbn_cuda_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream) {
    if (bytes == 0) return TBN_SUCCESS;
    TBN_REQUIRE(d_dst && d_src, TBN_INVALID_ARGUMENT, "tbn_cuda_d2d: null pointer");
    TBN_CUDA_TRY(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return TBN_SUCCESS;
}

int32_t tbn_cuda_sync(void* stream) {
    TBN_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    int dev = 0;
    TBN_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < kMaxDevices && g_dev[dev].ready) {
        volatile int* w = g_dev[dev].err_host;
        const int code = w[0];
        if (code != 0) {
            w[0] = 0;
            return fail(TBN_CUDA_TIMEOUT, "a bounded device-side wait expired (code " +
                                              std::to_string(code) + ") and the kernel gave up");
        }
    }
    return TBN_SUCCESS;
}

int32_t tbn_cuda_set_wait_limit_ns(uint64_t limit_ns) {
    TBN_REQUIRE(limit_ns >= 1000 && limit_ns <= 60000000000ull, TBN_INVALID_ARGUMENT,
                "tbn_cuda_set_wait_limit_ns: the limit must lie between 1 microsecond and 60 seconds");
    int dev = 0;
    TBN_CUDA_TRY(cudaGetDevice(&dev));
    TBN_REQUIRE(dev >= 0 && dev < kMaxDevices && g_dev[dev].ready, TBN_RUNTIME_ERROR,
                "tbn_cuda_init was not called on this device");
    *reinterpret_cast<volatile uint64_t*>(g_dev[dev].err_host + ptx::kWaitLimitWordOffset) = limit_ns;
    return TBN_SUCCESS;
}


int32_t tbn_cuda_selftest_wait_timeout(void* stream) {
    int* w = device_error_word();
    TBN_REQUIRE(w != nullptr, TBN_RUNTIME_ERROR, "tbn_cuda_init was not called on this device");
    wait_selftest_kernel<<<1, 32, 0, as_stream(stream)>>>(w);
    return launched("wait_selftest_kernel");
}

int64_t tbn_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int32_t tbn_cuda_profile_enable(int32_t enable) {
    g_profile.store(enable != 0, std::memory_order_relaxed);
    return TBN_SUCCESS;
}

int32_t tbn_cuda_profile_read(double* gemm_ms, int64_t* gemm_launches, double* split_ms, int64_t* split_launches) {
    double ms[2] = {0.0, 0.0};
    int64_t n[2] = {0, 0};
    std::vector<ProfileSpan> spans;
    {
        std::lock_guard<std::mutex> lock(g_prof_mutex);
        spans.swap(g_spans);
    }
    int32_t rc = TBN_SUCCESS;
    for (const ProfileSpan& s : spans) {
        float t = 0.0f;
        cudaError_t e = cudaEventSynchronize(s.stop);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, s.start, s.stop);
        if (e != cudaSuccess) rc = cuda_fail(e, "tbn_cuda_profile_read");
        else {
            ms[s.kind] += t;
            n[s.kind] += 1;
        }
        cudaEventDestroy(s.start);
        cudaEventDestroy(s.stop);
    }
    if (gemm_ms) *gemm_ms = ms[kProfGemm];
    if (gemm_launches) *gemm_launches = n[kProfGemm];
    if (split_ms) *split_ms = ms[kProfSplit];
    if (split_launches) *split_launches = n[kProfSplit];
    return rc;
}

int32_t tbn_packed_dims(int64_t K, int64_t N, int64_t* K_pad, int64_t* N_pad) {
    TBN_REQUIRE(K >= 0 && N >= 0 && K_pad && N_pad, TBN_INVALID_ARGUMENT, "tbn_packed_dims: bad arguments");
    *K_pad = round_up(K, 128);
    *N_pad = round_up(N, 8);
    return TBN_SUCCESS;
}

}  // extern "C"
