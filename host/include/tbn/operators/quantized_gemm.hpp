// Same include name as the reference; the declarations live in ops.hpp and, for the operators on pre-packed
// operands (qlinear_matmul_binary_blocked_packed / _blocked_prepacked), in gemm/packed_matrix.hpp.
#pragma once
#include "../gemm/packed_matrix.hpp"
#include "ops.hpp"
