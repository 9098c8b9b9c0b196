// Umbrella header of the tbn:: API (reference: tbn-runtime/include/tbn/tbn.hpp).
#pragma once
#include "onnx_integration/onnx_parser.hpp"
#include "gemm/packed_matrix.hpp"
#include "operators/ops.hpp"
#include "runtime/attribute.hpp"
#include "runtime/model.hpp"
#include "runtime/sharded_gemm.hpp"
#include "runtime/tensor.hpp"
#include "runtime/types.hpp"
#include "utils/errors.hpp"
