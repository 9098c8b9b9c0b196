// tbn::ShardedGemm: bookkeeping of the column-sharded multi-GPU GEMM over the C ABI.
#include "tbn/runtime/sharded_gemm.hpp"

#include <string>

#include "tbn_cuda.h"

namespace tbn {

namespace detail {
void ensure_runtime();
}

ShardedGemm::ShardedGemm(int rank, int world, std::int64_t M, std::int64_t K, std::int64_t N)
    : rank_(rank), world_(world), M_(M), K_(K), N_(N) {
    TBN_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world, InvalidArgumentError, "ShardedGemm: bad rank / world size");
    TBN_CHECK(M > 0 && K > 0 && N > 0, InvalidShapeError, "ShardedGemm: dimensions must be positive");
    TBN_CHECK(N % world == 0 && (N / world) % 4 == 0 && N % 4 == 0, InvalidShapeError,
              "ShardedGemm: N must divide evenly over the ranks into slabs that are multiples of 4 columns");
    detail::ensure_runtime();
    c0_ = rank * (N / world);
    c1_ = c0_ + N / world;
    c_ = Tensor(Shape{M, N}, DataType::FLOAT32, DeviceType::CUDA);
    (void)c_.device_data();
    opened_.assign(static_cast<size_t>(world), nullptr);
}

ShardedGemm::~ShardedGemm() {
    for (void* p : opened_)
        if (p) tbn_ipc_close(p);
}

std::vector<int> ShardedGemm::destination_ranks() const {
    std::vector<int> order;
    for (int i = 0; i < world_; ++i) order.push_back((rank_ + i) % world_);
    return order;
}

void ShardedGemm::set_weights(const Tensor& w_slab, float threshold) {
    TBN_CHECK(w_slab.shape().dims == std::vector<std::int64_t>({K_, c1_ - c0_}), InvalidShapeError,
              "ShardedGemm: the weight slab must be [K, N / world]");
    w_ = pack_binary_weights(w_slab, threshold, false);
}

void ShardedGemm::set_weights_ternary(const Tensor& w_slab, float lo, float hi) {
    TBN_CHECK(w_slab.shape().dims == std::vector<std::int64_t>({K_, c1_ - c0_}), InvalidShapeError,
              "ShardedGemm: the weight slab must be [K, N / world]");
    w_ = pack_ternary_weights(w_slab, lo, hi);
}

ShardedGemm::Handle ShardedGemm::export_result() const {
    Handle h{};
    detail::check(tbn_ipc_export(const_cast<void*>(c_.device_data()), h.data()));
    return h;
}

void ShardedGemm::connect(const std::vector<Handle>& handles) {
    TBN_CHECK(static_cast<int>(handles.size()) == world_, InvalidArgumentError, "ShardedGemm: one handle per rank is required");
    dests_.clear();
    for (int r : destination_ranks()) {
        float* base;
        if (r == rank_) {
            base = static_cast<float*>(c_.device_data());
        } else {
            if (!opened_[static_cast<size_t>(r)]) detail::check(tbn_ipc_open(handles[static_cast<size_t>(r)].data(), &opened_[static_cast<size_t>(r)]));
            base = static_cast<float*>(opened_[static_cast<size_t>(r)]);
        }
        dests_.push_back(base + c0_);
    }
}

void ShardedGemm::multiply(const Tensor& a, const Tensor* bias_slab, float scale) {
    TBN_CHECK(a.dtype() == DataType::FLOAT32 && a.shape().dims == std::vector<std::int64_t>({M_, K_}), InvalidShapeError,
              "ShardedGemm: A must be FLOAT32 [M, K]");
    TBN_CHECK(w_.N == c1_ - c0_ && w_.K == K_, RuntimeError, "ShardedGemm: set_weights first");
    if (dests_.empty()) {
        TBN_CHECK(world_ == 1, RuntimeError, "ShardedGemm: connect() the ranks first");
        dests_.push_back(static_cast<float*>(c_.device_data()));
    }
    const size_t ws_bytes = tbn_gemm_workspace_bytes(M_, K_, TBN_MODE_TC_BF16X2);
    Tensor ws = Tensor::device_uninitialized(Shape{static_cast<std::int64_t>(ws_bytes)}, DataType::UINT8);
    detail::check(tbn_gemm_fxb_multi(static_cast<const float*>(a.device_data()), M_, K_, K_,
                                     static_cast<const std::uint32_t*>(w_.neg.device_data()),
                                     w_.ternary ? static_cast<const std::uint32_t*>(w_.pos.device_data()) : nullptr, c1_ - c0_,
                                     static_cast<const float*>(w_.alpha.device_data()), scale,
                                     bias_slab ? static_cast<const float*>(bias_slab->device_data()) : nullptr, dests_.data(),
                                     static_cast<std::int32_t>(dests_.size()), N_, TBN_MODE_TC_BF16X2, 0, ws.device_data(), ws_bytes,
                                     nullptr));
    c_.mark_device_written();
    synchronize();   // the workspace above is released on return; the peers' copies still need the caller's barrier
}

}  // namespace tbn
