// Column-sharded float x binary GEMM across the GPUs of one box, one process per GPU.
//
// No counterpart in the reference (single device); it is the multi-GPU form of the product behind
// tbn::qlinear_matmul_binary / tbn::gemm on packed weights (tbn-runtime/include/tbn/operators/quantized_gemm.hpp:48-57).
// Rank g owns the weight columns [g*N/G, (g+1)*N/G) -- one contiguous range of packed words -- the activations are
// replicated, and ONE kernel per rank (tbn_gemm_fxb_multi) computes the slab and stores every finished tile into
// every rank's result matrix over NVLink: compute and all-gather fused.  The class owns the bookkeeping:
//   ShardedGemm sg(rank, world, M, K, N);            allocates this rank's C [M, N] on the current device
//   sg.set_weights(W_slab);                          packs this rank's columns (fp32 [K, N/G])
//   auto h = sg.export_result();                     64-byte handle; exchange all ranks' handles on the host
//   sg.connect(handles);                             opens the peers' matrices, builds the destination list
//   sg.multiply(A);                                  enqueues the fused kernel (A fp32 [M, K], the same on every rank)
//   <cross-process barrier after tbn::synchronize()> then sg.result() holds the whole product on every rank
// The cross-process barrier and the transport of the handles are the caller's (MPI, files, sockets ...).
#pragma once

#include <array>
#include <cstdint>
#include <utility>
#include <vector>

#include "../operators/ops.hpp"
#include "tensor.hpp"

namespace tbn {

class ShardedGemm {
public:
    using Handle = std::array<std::uint8_t, 64>;

    ShardedGemm(int rank, int world, std::int64_t M, std::int64_t K, std::int64_t N);
    ~ShardedGemm();
    ShardedGemm(const ShardedGemm&) = delete;
    ShardedGemm& operator=(const ShardedGemm&) = delete;

    // [begin, end) of the output columns this rank computes.
    std::pair<std::int64_t, std::int64_t> columns() const { return {c0_, c1_}; }
    // Order in which this rank's epilogue writes the ranks: itself first, then rank+1, rank+2, ... (ring order,
    // so that at any moment the ranks target different peers).
    std::vector<int> destination_ranks() const;

    void set_weights(const Tensor& w_slab, float threshold = 0.0f);   // fp32 [K, N / world]
    void set_weights_ternary(const Tensor& w_slab, float threshold_low, float threshold_high);
    Handle export_result() const;
    void connect(const std::vector<Handle>& handles);   // handles[r] of every rank r (this rank's own entry is ignored)
    void multiply(const Tensor& a, const Tensor* bias_slab = nullptr, float scale = 1.0f);
    Tensor& result() { return c_; }

private:
    int rank_, world_;
    std::int64_t M_, K_, N_, c0_, c1_;
    Tensor c_;
    PackedWeights w_;
    std::vector<void*> opened_;       // peers' matrices in this process's address space (index = rank; own = nullptr)
    std::vector<float*> dests_;       // destination list of the kernel, already offset to this rank's first column
};

}  // namespace tbn
