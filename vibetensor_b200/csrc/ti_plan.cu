// Host-side iteration planner and the library-wide plumbing (last error, validation).
#include "ti_plan.h"

#include <algorithm>
#include <atomic>
#include <mutex>

namespace vb {

std::string& last_error_ref() {
  thread_local std::string e;
  return e;
}

int sm_count(int device) {
  static std::mutex mu;
  static int cached[64];
  std::lock_guard<std::mutex> lk(mu);
  if (device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = 148;
    cached[device] = n;
  }
  return cached[device];
}

vbt_b200_status validate_tensor(const vbt_b200_tensor* t, const char* what) {
  VB_ARG(t != nullptr, std::string(what) + ": null tensor descriptor");
  VB_ARG(t->ndim >= 0, std::string(what) + ": negative rank");
  VB_ARG(itemsize(t->dtype) != 0, std::string(what) + ": unsupported dtype");
  VB_ARG(t->ndim == 0 || (t->sizes && t->strides), std::string(what) + ": null sizes/strides");
  for (int i = 0; i < t->ndim; ++i)
    VB_ARG(t->sizes[i] >= 0, std::string(what) + ": negative size");
  return VBT_B200_OK;
}

vbt_b200_status validate_data(const vbt_b200_tensor* t, const char* what) {
  VB_TRY(validate_tensor(t, what));
  VB_ARG(t->data != nullptr || numel(*t) == 0, std::string(what) + ": null data pointer");
  return VBT_B200_OK;
}

vbt_b200_launch_info& launch_info_ref() {
  thread_local vbt_b200_launch_info li{};
  return li;
}

namespace {
std::atomic<uint64_t> g_launches[VBT_B200_FAMILY_COUNT];
}
void count_launches(int family, int n) {
  if (family >= 0 && family < VBT_B200_FAMILY_COUNT && n > 0)
    g_launches[family].fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed);
}

vbt_b200_status broadcast_shape(const vbt_b200_tensor* const* ops, int n, const char* opname,
                                int64_t* out_sizes, int* out_ndim) {
  int nd = 0;
  for (int k = 0; k < n; ++k) {
    VB_TRY(validate_tensor(ops[k], opname));
    nd = std::max(nd, ops[k]->ndim);
  }
  if (nd > VBT_B200_MAX_NDIM)
    return fail(VBT_B200_INVALID_ARGUMENT,
                std::string(opname) + ": CUDA broadcast supports up to 25D (got " +
                    std::to_string(nd) + "D)");
  for (int d = 0; d < nd; ++d) out_sizes[d] = 1;
  for (int k = 0; k < n; ++k) {
    const int shift = nd - ops[k]->ndim;
    for (int d = 0; d < ops[k]->ndim; ++d) {
      const int64_t s = ops[k]->sizes[d];
      int64_t& o = out_sizes[d + shift];
      if (s == 1) continue;
      if (o == 1) o = s;
      else if (o != s)
        return fail(VBT_B200_INVALID_ARGUMENT,
                    std::string(opname) + ": shape mismatch: operands cannot be broadcast together");
    }
  }
  *out_ndim = nd;
  return VBT_B200_OK;
}

vbt_b200_status build_ti_plan(const vbt_b200_tensor* const* ops, int nops, const char* opname,
                              TiPlan* plan) {
  VB_ARG(nops >= 1 && nops <= kMaxOps, std::string(opname) + ": bad operand count");
  for (int k = 0; k < nops; ++k) VB_TRY(validate_tensor(ops[k], opname));
  const vbt_b200_tensor& out = *ops[0];
  if (out.ndim > VBT_B200_MAX_NDIM)
    return fail(VBT_B200_INVALID_ARGUMENT,
                std::string(opname) + ": CUDA broadcast supports up to 25D (got " +
                    std::to_string(out.ndim) + "D)");
  // the output must have exactly the broadcast shape of the inputs
  if (nops > 1) {
    int64_t bs[VBT_B200_MAX_NDIM];
    int bnd = 0;
    VB_TRY(broadcast_shape(ops + 1, nops - 1, opname, bs, &bnd));
    bool same = bnd == out.ndim;
    for (int d = 0; same && d < bnd; ++d) same = bs[d] == out.sizes[d];
    VB_ARG(same, std::string(opname) + ": output shape does not equal the broadcast shape of the inputs");
  }
  const int nd = out.ndim;
  plan->nops = nops;
  plan->numel = numel(out);
  for (int k = 0; k < nops; ++k) {
    plan->ptr[k] = static_cast<char*>(ops[k]->data);
    plan->esize[k] = itemsize(ops[k]->dtype);
  }
  if (plan->numel == 0) {
    plan->ndim = 0;
    return VBT_B200_OK;
  }
  for (int k = 0; k < nops; ++k)
    VB_ARG(ops[k]->data != nullptr, std::string(opname) + ": null data pointer");

  // per-dim strides in the output's index space (missing / size-1 dims broadcast with 0)
  struct Dim {
    int64_t size;
    int64_t st[kMaxOps];
    int order;
  };
  std::vector<Dim> dims;
  dims.reserve(nd);
  for (int d = 0; d < nd; ++d) {
    if (out.sizes[d] == 1) continue;
    Dim dm{};
    dm.size = out.sizes[d];
    dm.order = d;
    for (int k = 0; k < nops; ++k) {
      const int dk = d - (nd - ops[k]->ndim);
      dm.st[k] = (dk < 0 || ops[k]->sizes[dk] == 1) ? 0 : ops[k]->strides[dk];
    }
    VB_ARG(dm.st[0] != 0, std::string(opname) + ": output has internal overlap (stride 0)");
    dims.push_back(dm);
  }
  // walk every dim forwards in output memory
  for (auto& dm : dims) {
    if (dm.st[0] < 0) {
      for (int k = 0; k < nops; ++k) {
        plan->ptr[k] += (dm.size - 1) * dm.st[k] * plan->esize[k];
        dm.st[k] = -dm.st[k];
      }
    }
  }
  // dim 0 = smallest output stride; ties keep the original inner-most first
  std::stable_sort(dims.begin(), dims.end(), [](const Dim& a, const Dim& b) {
    if (a.st[0] != b.st[0]) return a.st[0] < b.st[0];
    return a.order > b.order;
  });
  // the output must not overlap itself: each stride clears the extent of the faster dims
  {
    int64_t extent = 1;
    for (const auto& dm : dims) {
      VB_ARG(dm.st[0] >= extent, std::string(opname) + ": output has internal overlap");
      extent += (dm.size - 1) * dm.st[0];
    }
  }
  // merge dim d+1 into d when every operand walks them as one
  std::vector<Dim> merged;
  for (const auto& dm : dims) {
    if (!merged.empty()) {
      Dim& p = merged.back();
      bool ok = true;
      for (int k = 0; k < nops && ok; ++k) ok = dm.st[k] == p.st[k] * p.size;
      if (ok) {
        p.size *= dm.size;
        continue;
      }
    }
    merged.push_back(dm);
  }
  if (merged.empty()) {  // a single element
    Dim one{};
    one.size = 1;
    for (int k = 0; k < nops; ++k) one.st[k] = k == 0 ? 1 : 0;
    merged.push_back(one);
  }
  plan->ndim = static_cast<int>(merged.size());
  for (int d = 0; d < plan->ndim; ++d) {
    plan->shape[d] = merged[d].size;
    for (int k = 0; k < nops; ++k) plan->stride[k][d] = merged[d].st[k];
  }
  // inputs that partially overlap the output would be read after being overwritten
  auto range = [&](int k, const char*& lo, const char*& hi) {
    lo = hi = plan->ptr[k];
    for (int d = 0; d < plan->ndim; ++d) {
      const int64_t span = (plan->shape[d] - 1) * plan->stride[k][d] * plan->esize[k];
      if (span >= 0) hi += span; else lo += span;
    }
    hi += plan->esize[k];
  };
  const char *olo, *ohi;
  range(0, olo, ohi);
  for (int k = 1; k < nops; ++k) {
    const char *ilo, *ihi;
    range(k, ilo, ihi);
    if (ilo < ohi && olo < ihi) {
      bool identical = plan->ptr[k] == plan->ptr[0] && plan->esize[k] == plan->esize[0];
      for (int d = 0; identical && d < plan->ndim; ++d)
        identical = plan->stride[k][d] == plan->stride[0][d];
      VB_ARG(identical, std::string(opname) + ": input partially overlaps the output");
    }
  }
  return VBT_B200_OK;
}

TiKernel choose_ti_kernel(const TiPlan& plan, int V, bool* flat_vec_ok) {
  auto aligned = [&](int k, int64_t elem_off) {
    return ((reinterpret_cast<uintptr_t>(plan.ptr[k]) + elem_off * plan.esize[k]) %
            (static_cast<uintptr_t>(V) * plan.esize[k])) == 0;
  };
  if (plan.ndim == 1) {
    bool flat = plan.stride[0][0] == 1;
    for (int k = 1; k < plan.nops && flat; ++k)
      flat = plan.stride[k][0] == 0 || plan.stride[k][0] == 1;
    if (flat) {
      bool vec = V > 1;
      for (int k = 0; k < plan.nops && vec; ++k)
        if (plan.stride[k][0] == 1) vec = aligned(k, 0);
      *flat_vec_ok = vec;
      return kTiFlat;
    }
  }
  *flat_vec_ok = false;
  // vector kernel: the output is contiguous along dim 0 in whole vectors, and every operand
  // that is contiguous along dim 0 starts each row on a vector boundary
  bool vec = V > 1 && plan.stride[0][0] == 1 && plan.shape[0] % V == 0;
  for (int k = 0; k < plan.nops && vec; ++k) {
    if (plan.stride[k][0] != 1) continue;
    vec = aligned(k, 0);
    for (int d = 1; d < plan.ndim && vec; ++d) vec = plan.stride[k][d] % V == 0;
  }
  return vec ? kTiTiledVec : kTiTiledScalar;
}

// Which inputs should go through the transposing kernel, and along which dim: an input
// qualifies when it would have to be gathered along dim 0, is contiguous along one other
// dim j, both extents are at least 16, and it really varies over the tensor (an input that is
// broadcast along a long dim is better served by the register-hoisting kernel above).
// Returns the mask (0 = none) and sets *dimj.
int transpose_candidates(const TiPlan& plan, int* dimj) {
  int mask = 0, jsel = -1;
  if (plan.ndim < 2 || plan.shape[0] < 16) return 0;
  for (int k = 1; k < plan.nops; ++k) {
    const int64_t s0 = plan.stride[k][0];
    if (s0 == 0 || s0 == 1 || s0 == -1) continue;
    int j = -1;
    bool broadcast_long = false;
    for (int d = 1; d < plan.ndim; ++d) {
      if (plan.stride[k][d] == 1 && plan.shape[d] >= 16 && j < 0) j = d;
      if (plan.stride[k][d] == 0 && plan.shape[d] >= 16) broadcast_long = true;
    }
    if (j < 0 || broadcast_long) continue;
    if (jsel >= 0 && j != jsel) continue;  // one partner dim per launch
    jsel = j;
    mask |= 1 << (k - 1);
  }
  *dimj = jsel;
  return mask;
}

}  // namespace vb

extern "C" {

const char* vbt_b200_last_error(void) { return vb::last_error_ref().c_str(); }
int32_t vbt_b200_version(void) { return 1000; }
int32_t vbt_b200_compiled_arch(void) { return 100; }

vbt_b200_status vbt_b200_last_launch_info(vbt_b200_launch_info* out) {
  VB_ARG(out != nullptr, "last_launch_info: null argument");
  *out = vb::launch_info_ref();
  return VBT_B200_OK;
}

void vbt_b200_reset_last_launch_info(void) { vb::launch_info_ref() = vbt_b200_launch_info{}; }

vbt_b200_status vbt_b200_launch_counts(uint64_t* counts, int32_t n) {
  VB_ARG(counts != nullptr && n >= 0, "launch_counts: bad argument");
  for (int i = 0; i < n; ++i)
    counts[i] = i < VBT_B200_FAMILY_COUNT ? vb::g_launches[i].load(std::memory_order_relaxed) : 0;
  return VBT_B200_OK;
}

void vbt_b200_reset_launch_counts(void) {
  for (auto& c : vb::g_launches) c.store(0, std::memory_order_relaxed);
}

vbt_b200_status vbt_b200_enable_peer_access(int32_t compute_device, int32_t peer_device) {
  using namespace vb;
  int n = 0;
  VB_CUDA(cudaGetDeviceCount(&n));
  VB_ARG(compute_device >= 0 && compute_device < n && peer_device >= 0 && peer_device < n,
         "[Fabric] enable_peer_access: device index out of range");
  if (compute_device == peer_device) return VBT_B200_OK;
  int can = 0;
  VB_CUDA(cudaDeviceCanAccessPeer(&can, compute_device, peer_device));
  VB_REQUIRE(can != 0, VBT_B200_RUNTIME_ERROR,
             "[Fabric] device " + std::to_string(compute_device) + " cannot access device " +
                 std::to_string(peer_device) + " memory (no P2P path)");
  int prev = 0;
  VB_CUDA(cudaGetDevice(&prev));
  VB_CUDA(cudaSetDevice(compute_device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // not an error: somebody (the host framework) enabled it before
    e = cudaSuccess;
  }
  cudaSetDevice(prev);
  if (e != cudaSuccess)
    return fail(VBT_B200_CUDA_ERROR, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_broadcast_shape(const vbt_b200_tensor* const* operands, int32_t n,
                                         int64_t* out_sizes, int32_t* out_ndim) {
  VB_ARG(operands && out_sizes && out_ndim && n >= 1, "broadcast_shape: null argument");
  int nd = 0;
  VB_TRY(vb::broadcast_shape(operands, n, "broadcast_shape", out_sizes, &nd));
  *out_ndim = nd;
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_ti_plan(const vbt_b200_tensor* const* operands, int32_t noperands,
                                 int64_t* shape, int64_t* strides, int32_t* ndim, int32_t* kernel,
                                 int32_t* pieces) {
  VB_ARG(operands && shape && strides && ndim && kernel && pieces, "ti_plan: null argument");
  vb::TiPlan plan;
  VB_TRY(vb::build_ti_plan(operands, noperands, "ti_plan", &plan));
  *ndim = plan.ndim;
  for (int d = 0; d < plan.ndim; ++d) {
    shape[d] = plan.shape[d];
    for (int k = 0; k < noperands; ++k) strides[k * VBT_B200_MAX_NDIM + d] = plan.stride[k][d];
  }
  bool flat_vec = false;
  const int V = plan.esize[0] > 0 ? 16 / std::max(plan.esize[0], plan.nops > 1 ? plan.esize[1] : 1) : 1;
  *kernel = plan.numel == 0 ? 0 : static_cast<int>(vb::choose_ti_kernel(plan, V, &flat_vec));
  int dimj = -1;
  if (*kernel != 0 && vb::transpose_candidates(plan, &dimj) != 0) *kernel = 3;
  *pieces = 1;
  return VBT_B200_OK;
}

}  // extern "C"
