// Per-shape choice of the GEMM kernel variant.  Stands in for the reference's TilingParams / auto_tune_gemm
// (GeMM/05-final/GeMM.hpp:16-43, tbn-runtime/src/operators/gemm.cpp:524-536): there the caller hands tile sizes
// to a CPU engine; here a table measured on the GPU (CUDA-event sweep, fast_arm_tbcnn_b200/tune.py) is compiled
// into the library and TBN_MODE_AUTO looks the shape's class up in it.
#pragma once

#include <cstdint>

namespace tbn_cuda {

struct GemmPlan {
    int kernel;       // 0: tcgen05 tensor-core kernel, 1: CUDA-core add/subtract-by-sign kernel,
                      // 2: tcgen05 on CTA pairs (cta_group::2, 256 x 256 tiles; large products)
    int bn;           // column tile of the tensor-core kernel: 64, 128 or 256
    int group_m;      // rasterisation group: m-tiles that share one sweep over the column tiles
    int fused_split;  // 1: the GEMM kernel reads the fp32 rows and splits them in registers (no separate split pass)
};

constexpr int kPlanClassesM = 6, kPlanClassesN = 6, kPlanClassesK = 4;
int plan_class_m(int64_t M);
int plan_class_n(int64_t N);
int plan_class_k(int64_t K);
// Table entry of the shape's class, adjusted to the shape (tile padding), with any override applied.
GemmPlan gemm_plan(int64_t M, int64_t N, int64_t K);

}  // namespace tbn_cuda
