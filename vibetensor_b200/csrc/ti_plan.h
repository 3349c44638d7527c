// Host-side iteration planner for elementwise ops over broadcast / strided views.
//
// Does for this library what TensorIterConfig::build does for the reference's elementwise
// branch (src/vbt/core/tensor_iterator/core.cc:1121-1916): broadcast every operand to the
// output shape, drop size-1 dims, order dims by ascending |output stride| so that dim 0 is
// the one the output is (most) contiguous in, flip dims the output walks backwards, and
// merge adjacent dims that every operand walks as one.  The result feeds the kernels'
// offset calculator, which replaces compute_offset_elems
// (include/vbt/core/tensor_iterator/cuda.h:25-42).
#pragma once
#include "common.cuh"

namespace vb {

constexpr int kMaxOps = 4;

struct TiPlan {
  int nops{0};
  int ndim{0};                              // after coalescing; >= 1 unless numel == 0
  int64_t numel{0};
  int64_t shape[VBT_B200_MAX_NDIM]{};       // innermost (dim 0) first
  int64_t stride[kMaxOps][VBT_B200_MAX_NDIM]{};  // elements, per operand (0 = out)
  char* ptr[kMaxOps]{};                     // base pointers after negative-stride flips
  int esize[kMaxOps]{};
};

// ops[0] is the output.  `opname` prefixes error messages ("vt::add").
vbt_b200_status build_ti_plan(const vbt_b200_tensor* const* ops, int nops, const char* opname,
                              TiPlan* plan);

// Shape of the broadcast of n operands (right-aligned; sizes must match or be 1).
vbt_b200_status broadcast_shape(const vbt_b200_tensor* const* ops, int n, const char* opname,
                                int64_t* out_sizes, int* out_ndim);

// Kernel selection for a plan with vector width V elements of the output type.
enum TiKernel { kTiFlat = 0, kTiTiledVec = 1, kTiTiledScalar = 2 };
// vec_bytes[k] = bytes one vector of operand k spans (V * esize[k]).
TiKernel choose_ti_kernel(const TiPlan& plan, int V, bool* flat_vec_ok);

// Inputs (bit k-1 = input k) that the shared-memory transposing kernel should stage, and the
// iteration dim they are contiguous in; 0 = use the kernels above.
int transpose_candidates(const TiPlan& plan, int* dimj);

}  // namespace vb
