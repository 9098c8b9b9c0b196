// tbn::Tensor with device residency.
//
// Same surface as the reference's Tensor (tbn-runtime/include/tbn/runtime/tensor.hpp:11-110):
// shape / dtype / device / data() / typed_data<T>() / num_elements() / copy() / to_device(), copies
// alias the same storage, construction zero-fills.  New: a tensor may live in HBM
// (DeviceType::CUDA).  The storage keeps a device buffer and a host mirror and moves data lazily:
// typed_data() / data() hand out the host mirror (downloading first if the device copy is newer);
// device_data() hands out the device buffer (uploading first if the host copy is newer).
// A mutable host pointer marks the device copy stale.  Not thread-safe, like the reference.
// Device buffers come from a caching pool (the Session's tensor allocator, now in HBM): a freed block is kept and
// handed to the next request of a similar size, so that a Session run allocates from the driver only while its
// working set still grows.  All kernels of this layer run on one stream, which orders reuse after the last use.
#pragma once

#include <memory>
#include <vector>

#include "../utils/errors.hpp"
#include "types.hpp"

namespace tbn {

namespace detail {
struct Storage {
    size_t bytes = 0;
    size_t capacity = 0;  // bytes of the device block (a pooled block may be larger than `bytes`)
    std::unique_ptr<uint8_t[]> host;
    void* device = nullptr;
    bool host_valid = false;
    bool device_valid = false;
    ~Storage();
};
}  // namespace detail

class Tensor {
public:
    Tensor() = default;
    Tensor(const Shape& shape, DataType dtype, DeviceType device = DeviceType::CPU);
    Tensor(const Shape& shape, DataType dtype, const void* data, DeviceType device = DeviceType::CPU);
    // Device tensor whose contents are NOT zero-filled: for results that a kernel overwrites completely.
    static Tensor device_uninitialized(const Shape& shape, DataType dtype);

    const Shape& shape() const { return shape_; }
    DataType dtype() const { return dtype_; }
    DeviceType device() const { return device_; }
    size_t data_size() const { return storage_ ? storage_->bytes : 0; }
    int64_t num_elements() const { return shape_.dims.empty() ? 1 : shape_.size(); }
    int64_t dim(int idx) const {
        TBN_CHECK(idx >= 0 && idx < static_cast<int>(shape_.dims.size()), InvalidArgumentError,
                  "Dimension index out of range");
        return shape_.dims[idx];
    }

    // Host view (synchronises the host mirror first).
    void* data();
    const void* data() const;
    template <typename T> T* typed_data() { return static_cast<T*>(data()); }
    template <typename T> const T* typed_data() const { return static_cast<const T*>(data()); }

    // Device view (allocates / uploads on first use).  The const form promises not to write.
    void* device_data();
    const void* device_data() const;
    // Tells the storage that a kernel wrote the device buffer (host mirror becomes stale).
    void mark_device_written();

    const QuantizationParams& quantization_params() const { return qparams_; }
    void set_quantization_params(const QuantizationParams& p) { qparams_ = p; }

    Tensor copy() const;                        // deep copy, same residency
    Tensor to_device(DeviceType device) const;  // deep copy with the requested residency
    Tensor reshaped(const Shape& shape) const;  // alias with another shape (same element count)
    bool empty() const { return !storage_; }

private:
    Shape shape_;
    DataType dtype_ = DataType::FLOAT32;
    DeviceType device_ = DeviceType::CPU;
    std::shared_ptr<detail::Storage> storage_;
    QuantizationParams qparams_;
    void ensure_host() const;
    void ensure_device() const;
};

Tensor make_tensor(const Shape& shape, const std::vector<float>& data);
Tensor make_tensor(const Shape& shape, const std::vector<TernaryWeight>& data);
Tensor make_tensor(const Shape& shape, const std::vector<BinaryWeight>& data);

}  // namespace tbn
