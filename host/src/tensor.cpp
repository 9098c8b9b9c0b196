// tbn::Tensor storage on top of the C ABI (tbn_cuda_malloc / h2d / d2h), error mapping, helpers.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>

#include "tbn/runtime/tensor.hpp"
#include "tbn_cuda.h"

namespace tbn {

namespace detail {

void throw_status(int status) {
    char msg[1024];
    tbn_cuda_last_error(msg, sizeof msg);
    switch (status) {
        case TBN_INVALID_ARGUMENT: throw InvalidArgumentError(msg);
        case TBN_OUT_OF_MEMORY: throw OutOfMemoryError(msg);
        case TBN_NOT_IMPLEMENTED: throw NotImplementedError(msg);
        case TBN_INVALID_SHAPE: throw InvalidShapeError(msg);
        default: throw RuntimeError(std::string(msg) + " (status " + std::to_string(status) + ")");
    }
}

void ensure_runtime() {
    static std::once_flag once;
    static int status = 0;
    // One process drives one GPU: device 0 unless TBN_DEVICE names another (one process per GPU on a multi-GPU box).
    std::call_once(once, [] {
        const char* dev = std::getenv("TBN_DEVICE");
        status = tbn_cuda_init(dev ? std::atoi(dev) : 0);
    });
    check(status);
}

// Caching pool of device blocks.  Requests are rounded up to 512 bytes; a cached block is reused when it is at
// most twice the request (or within 1 MiB of it); at most kPoolLimit bytes stay cached.
class DevicePool {
public:
    void* acquire(size_t bytes, bool zero, size_t* capacity) {
        const size_t want = (bytes + 511) / 512 * 512;
        {
            std::lock_guard<std::mutex> lock(mutex_);
            auto it = free_.lower_bound(want);
            if (it != free_.end() && it->first <= std::max(want * 2, want + (size_t(1) << 20))) {
                void* p = it->second;
                *capacity = it->first;
                cached_ -= it->first;
                free_.erase(it);
                if (zero) check(tbn_cuda_memset(p, 0, bytes, nullptr));
                return p;
            }
        }
        void* p = nullptr;
        const int status = tbn_cuda_malloc(&p, want);  // zero-filled by the library
        if (status == TBN_OUT_OF_MEMORY) {           // give the cached blocks back and try once more
            trim(0);
            check(tbn_cuda_malloc(&p, want));
        } else {
            check(status);
        }
        *capacity = want;
        return p;
    }
    void release(void* p, size_t capacity) {
        if (!p) return;
        {
            std::lock_guard<std::mutex> lock(mutex_);
            if (cached_ + capacity <= kPoolLimit) {
                free_.emplace(capacity, p);
                cached_ += capacity;
                return;
            }
        }
        tbn_cuda_free(p);
    }
    void trim(size_t keep) {
        std::lock_guard<std::mutex> lock(mutex_);
        while (cached_ > keep && !free_.empty()) {
            auto it = std::prev(free_.end());
            tbn_cuda_free(it->second);
            cached_ -= it->first;
            free_.erase(it);
        }
    }

private:
    static constexpr size_t kPoolLimit = size_t(32) << 30;
    std::mutex mutex_;
    std::multimap<size_t, void*> free_;
    size_t cached_ = 0;
};

DevicePool& pool() {
    static DevicePool* p = new DevicePool();  // never destroyed: the CUDA context may be gone at exit
    return *p;
}

Storage::~Storage() {
    if (device) pool().release(device, capacity);
}

}  // namespace detail

std::string shape_to_string(const Shape& shape) {
    std::ostringstream os;
    os << "[";
    for (size_t i = 0; i < shape.dims.size(); ++i) os << (i ? ", " : "") << shape.dims[i];
    os << "]";
    return os.str();
}

Tensor::Tensor(const Shape& shape, DataType dtype, DeviceType device)
    : shape_(shape), dtype_(dtype), device_(device), storage_(std::make_shared<detail::Storage>()) {
    for (int64_t d : shape.dims) TBN_CHECK(d >= 0, InvalidShapeError, "negative dimension in " + shape_to_string(shape));
    storage_->bytes = static_cast<size_t>(shape.size()) * element_size(dtype);
    if (device == DeviceType::CUDA) {
        detail::ensure_runtime();
        if (storage_->bytes) storage_->device = detail::pool().acquire(storage_->bytes, /*zero=*/true, &storage_->capacity);
        storage_->device_valid = true;
    } else {
        storage_->host.reset(new uint8_t[storage_->bytes ? storage_->bytes : 1]);
        std::memset(storage_->host.get(), 0, storage_->bytes);
        storage_->host_valid = true;
    }
}

Tensor::Tensor(const Shape& shape, DataType dtype, const void* data, DeviceType device) : Tensor(shape, dtype, DeviceType::CPU) {
    TBN_CHECK(data != nullptr || storage_->bytes == 0, InvalidArgumentError, "Tensor: null data pointer");
    if (storage_->bytes) std::memcpy(storage_->host.get(), data, storage_->bytes);
    device_ = device;
    if (device == DeviceType::CUDA) ensure_device();
}

Tensor Tensor::device_uninitialized(const Shape& shape, DataType dtype) {
    Tensor t;
    for (int64_t d : shape.dims) TBN_CHECK(d >= 0, InvalidShapeError, "negative dimension in " + shape_to_string(shape));
    t.shape_ = shape;
    t.dtype_ = dtype;
    t.device_ = DeviceType::CUDA;
    t.storage_ = std::make_shared<detail::Storage>();
    t.storage_->bytes = static_cast<size_t>(shape.size()) * element_size(dtype);
    detail::ensure_runtime();
    if (t.storage_->bytes) t.storage_->device = detail::pool().acquire(t.storage_->bytes, /*zero=*/false, &t.storage_->capacity);
    t.storage_->device_valid = true;
    return t;
}

void Tensor::ensure_host() const {
    TBN_CHECK(storage_ != nullptr, RuntimeError, "Tensor has no storage");
    detail::Storage& s = *storage_;
    if (s.host_valid) return;
    if (!s.host) s.host.reset(new uint8_t[s.bytes ? s.bytes : 1]);
    if (s.device_valid && s.bytes) {
        detail::check(tbn_cuda_d2h(s.host.get(), s.device, s.bytes, nullptr));
        detail::check(tbn_cuda_sync(nullptr));
    }
    s.host_valid = true;
}

void Tensor::ensure_device() const {
    TBN_CHECK(storage_ != nullptr, RuntimeError, "Tensor has no storage");
    detail::Storage& s = *storage_;
    if (s.device_valid) return;
    detail::ensure_runtime();
    if (!s.device && s.bytes) s.device = detail::pool().acquire(s.bytes, /*zero=*/!s.host_valid, &s.capacity);
    if (s.host_valid && s.bytes) {
        detail::check(tbn_cuda_h2d(s.device, s.host.get(), s.bytes, nullptr));
        detail::check(tbn_cuda_sync(nullptr));  // the host mirror may be freed or rewritten right after
    }
    s.device_valid = true;
}

void* Tensor::data() {
    ensure_host();
    storage_->device_valid = false;  // the caller may write through this pointer
    return storage_->host.get();
}

const void* Tensor::data() const {
    ensure_host();
    return storage_->host.get();
}

void* Tensor::device_data() {
    ensure_device();
    storage_->host_valid = false;
    return storage_->device;
}

const void* Tensor::device_data() const {
    ensure_device();
    return storage_->device;
}

void Tensor::mark_device_written() {
    if (storage_) {
        storage_->device_valid = true;
        storage_->host_valid = false;
    }
}

Tensor Tensor::copy() const { return to_device(device_); }

Tensor Tensor::to_device(DeviceType device) const {
    Tensor out(shape_, dtype_, device);
    out.qparams_ = qparams_;
    if (!storage_ || storage_->bytes == 0) return out;
    if (device == DeviceType::CUDA && storage_->device_valid) {
        detail::check(tbn_cuda_d2d(out.storage_->device, storage_->device, storage_->bytes, nullptr));
        out.mark_device_written();
    } else if (device == DeviceType::CUDA) {
        detail::check(tbn_cuda_h2d(out.storage_->device, data(), storage_->bytes, nullptr));
        detail::check(tbn_cuda_sync(nullptr));
        out.mark_device_written();
    } else {
        std::memcpy(out.storage_->host.get(), data(), storage_->bytes);
    }
    return out;
}

Tensor Tensor::reshaped(const Shape& shape) const {
    TBN_CHECK(shape.size() == num_elements(), InvalidShapeError,
              "cannot view " + shape_to_string(shape_) + " as " + shape_to_string(shape));
    Tensor out = *this;
    out.shape_ = shape;
    return out;
}

namespace {
template <typename T>
Tensor make_tensor_impl(const Shape& shape, const std::vector<T>& data, DataType dt) {
    TBN_CHECK(static_cast<int64_t>(data.size()) == shape.size(), InvalidShapeError, "Data size doesn't match shape");
    return Tensor(shape, dt, data.data());
}
}  // namespace

Tensor make_tensor(const Shape& shape, const std::vector<float>& data) { return make_tensor_impl(shape, data, DataType::FLOAT32); }
Tensor make_tensor(const Shape& shape, const std::vector<TernaryWeight>& data) { return make_tensor_impl(shape, data, DataType::TERNARY); }
Tensor make_tensor(const Shape& shape, const std::vector<BinaryWeight>& data) { return make_tensor_impl(shape, data, DataType::BINARY); }

}  // namespace tbn
