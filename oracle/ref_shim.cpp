// TEST INFRASTRUCTURE ONLY. This file is the thin C shim that is linked against
// VibeTensor's *own* CPU sources (compiled where they lie, never copied) to
// produce oracle/_ref/libvbt_ref_cpu.so.  Nothing in the product path may load
// it; only tests/, the smoke check and the bench's CPU-baseline leg do.
//
// Every entry wraps caller memory in a reference TensorImpl (no copy), calls
// the reference's CPU implementation and writes into a caller buffer:
//   * sum / mean        -> vbt_default_sum_impl / vbt_default_mean_impl
//                          (src/vbt/ops/default_kernels.cc:748-870)
//   * amax / argmax     -> TensorIter::reduce_op + for_each_reduction_cpu
//                          (src/vbt/core/tensor_iterator/core.cc:1980-2076,
//                           src/vbt/cpu/tensor_iterator/reduction.cc:176-329)
//                          driving loop callbacks that restate
//                          src/vbt/python/tensor_bindings.cc:361-379,:630-655
//                          (that TU needs nanobind and cannot be compiled here)
//   * binary / compare  -> Dispatcher::callBoxed("vt::<op>") CPU kernels
//                          (src/vbt/ops/default_kernels.cc:164-981)
//   * index / index_put_-> vbt::core::indexing::index / index_put_
//                          (src/vbt/core/indexing_advanced.cc:1474-1552)
//   * embedding         -> boxed "vt::embedding" CPU kernel
//                          (src/vbt/ops/embedding_dispatch.cc:292-533)
#include <cstdint>
#include <cstring>
#include <limits>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "vbt/core/indexing.h"
#include "vbt/core/tensor.h"
#include "vbt/core/tensor_iter.h"
#include "vbt/core/tensor_iterator/cpu.h"
#include "vbt/core/tensor_ops.h"
#include "vbt/core/view_ops.h"
#include "vbt/dispatch/dispatcher.h"

using vbt::core::ScalarType;
using vbt::core::TensorImpl;

TensorImpl vbt_default_sum_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim);
TensorImpl vbt_default_mean_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim);
extern "C" void vbt_register_default_kernels();
extern "C" void vbt_register_embedding_kernels();

namespace {

thread_local std::string g_err;

TensorImpl wrap(const void* data, int dtype, int ndim, const int64_t* sizes,
                const int64_t* strides) {
  std::vector<int64_t> sz(sizes, sizes + ndim), st(strides, strides + ndim);
  const auto dt = static_cast<ScalarType>(dtype);
  // Extent in elements of the addressed region (non-negative strides only).
  int64_t extent = 1;
  bool empty = false;
  for (int i = 0; i < ndim; ++i) {
    if (sz[i] == 0) empty = true;
    if (st[i] < 0) throw std::invalid_argument("ref shim: negative strides unsupported");
    extent += (sz[i] - 1) * st[i];
  }
  if (empty) extent = 0;
  const std::size_t nbytes = static_cast<std::size_t>(extent) * vbt::core::itemsize(dt);
  auto storage = vbt::core::make_intrusive<vbt::core::Storage>(
      vbt::core::DataPtr(const_cast<void*>(data), [](void*) {}), nbytes);
  return TensorImpl(storage, sz, st, 0, dt, vbt::core::Device::cpu());
}

// Copy a (contiguous) reference result into the caller's dense buffer.
void export_dense(const TensorImpl& t, void* out) {
  TensorImpl c = t.is_contiguous() ? t : vbt::core::clone_cpu(t);
  const std::size_t n = static_cast<std::size_t>(c.numel()) * c.itemsize();
  if (n) std::memcpy(out, c.data(), n);
}

template <class F>
int guarded(F&& f) {
  try {
    f();
    g_err.clear();
    return 0;
  } catch (const std::out_of_range& e) {
    g_err = e.what();
    return 3;
  } catch (const std::invalid_argument& e) {
    g_err = e.what();
    return 1;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 2;
  }
}

// Loop callbacks with the behaviour of tensor_bindings.cc:361-379 / :630-655:
// start from element 0, update on strict '>', first maximum wins.
void amax_f32(char** d, const int64_t* s, int64_t n, void*) {
  float best = *reinterpret_cast<const float*>(d[1]);
  for (int64_t i = 1; i < n; ++i) {
    float v = *reinterpret_cast<const float*>(d[1] + i * s[1]);
    if (v > best) best = v;
  }
  *reinterpret_cast<float*>(d[0]) = best;
}
void amax_i64(char** d, const int64_t* s, int64_t n, void*) {
  long long best = *reinterpret_cast<const long long*>(d[1]);
  for (int64_t i = 1; i < n; ++i) {
    long long v = *reinterpret_cast<const long long*>(d[1] + i * s[1]);
    if (v > best) best = v;
  }
  *reinterpret_cast<long long*>(d[0]) = best;
}
void amin_f32(char** d, const int64_t* s, int64_t n, void*) {
  float best = *reinterpret_cast<const float*>(d[1]);
  for (int64_t i = 1; i < n; ++i) {
    float v = *reinterpret_cast<const float*>(d[1] + i * s[1]);
    if (v < best) best = v;
  }
  *reinterpret_cast<float*>(d[0]) = best;
}
void argmax_f32(char** d, const int64_t* s, int64_t n, void*) {
  float best = *reinterpret_cast<const float*>(d[2]);
  int64_t bi = 0;
  for (int64_t i = 1; i < n; ++i) {
    float v = *reinterpret_cast<const float*>(d[2] + i * s[2]);
    if (v > best) { best = v; bi = i; }
  }
  *reinterpret_cast<float*>(d[0]) = best;
  *reinterpret_cast<long long*>(d[1]) = bi;
}
void argmax_i64(char** d, const int64_t* s, int64_t n, void*) {
  long long best = *reinterpret_cast<const long long*>(d[2]);
  int64_t bi = 0;
  for (int64_t i = 1; i < n; ++i) {
    long long v = *reinterpret_cast<const long long*>(d[2] + i * s[2]);
    if (v > best) { best = v; bi = i; }
  }
  *reinterpret_cast<long long*>(d[0]) = best;
  *reinterpret_cast<long long*>(d[1]) = bi;
}

TensorImpl new_dense(const std::vector<int64_t>& sizes, ScalarType dt, std::vector<char>& hold) {
  int64_t n = 1;
  for (auto s : sizes) n *= s;
  hold.assign(static_cast<std::size_t>(n) * vbt::core::itemsize(dt) + 16, 0);
  std::vector<int64_t> st(sizes.size());
  int64_t acc = 1;
  for (int i = static_cast<int>(sizes.size()) - 1; i >= 0; --i) { st[i] = acc; acc *= sizes[i]; }
  auto storage = vbt::core::make_intrusive<vbt::core::Storage>(
      vbt::core::DataPtr(hold.data(), [](void*) {}), hold.size());
  return TensorImpl(storage, sizes, st, 0, dt, vbt::core::Device::cpu());
}

void ensure_registered() {
  static bool once = [] {
    vbt_register_default_kernels();
    vbt_register_embedding_kernels();
    return true;
  }();
  (void)once;
}

}  // namespace

extern "C" {

const char* vref_last_error() { return g_err.c_str(); }

// kind: 0 sum, 1 mean.  dims may be empty (reduce all).  out is dense.
int vref_sum_mean(int kind, const void* x, int dtype, int ndim, const int64_t* sizes,
                  const int64_t* strides, const int64_t* dims, int ndims, int keepdim,
                  void* out) {
  return guarded([&] {
    TensorImpl t = wrap(x, dtype, ndim, sizes, strides);
    std::vector<int64_t> dv(dims, dims + ndims);
    TensorImpl r = kind == 0 ? vbt_default_sum_impl(t, dv, keepdim != 0)
                             : vbt_default_mean_impl(t, dv, keepdim != 0);
    export_dense(r, out);
  });
}

// kind: 0 amax, 1 amin, 2 argmax (values + int64 indices).  Single dim, as the
// reference's Python binding takes; dim == INT64_MIN means "all" (flattened).
// Non-contiguous input is cloned first (tensor_bindings.cc:469-472, :562-565).
int vref_minmax(int kind, const void* x, int dtype, int ndim, const int64_t* sizes,
                const int64_t* strides, int64_t dim, void* out_values, int64_t* out_indices) {
  return guarded([&] {
    TensorImpl self = wrap(x, dtype, ndim, sizes, strides);
    TensorImpl base = self.is_contiguous() ? self : vbt::core::clone_cpu(self);
    const auto dt = static_cast<ScalarType>(dtype);
    std::vector<int64_t> out_sizes;
    int64_t rd = 0;
    if (dim == std::numeric_limits<int64_t>::min()) {
      base = vbt::core::view(base, std::vector<int64_t>{base.numel()});
    } else {
      rd = dim < 0 ? dim + ndim : dim;
      if (rd < 0 || rd >= ndim) throw std::invalid_argument("reduction dim out of range");
      for (int d = 0; d < ndim; ++d)
        if (d != rd) out_sizes.push_back(sizes[d]);
    }
    int64_t on = 1;
    for (auto s : out_sizes) on *= s;
    if (on == 0) return;
    if (base.numel() == 0) throw std::runtime_error(kind == 1 ? "amin: empty" : "amax: empty");
    std::vector<char> hv, hi;
    TensorImpl vals = new_dense(out_sizes, dt, hv);
    if (kind == 2) {
      TensorImpl idx = new_dense(out_sizes, ScalarType::Int64, hi);
      auto iter = vbt::core::TensorIter::reduce_op(vals, idx, base,
                                                    std::span<const int64_t>(&rd, 1));
      vbt::core::for_each_reduction_cpu(iter, dt == ScalarType::Float32 ? &argmax_f32 : &argmax_i64,
                                        nullptr);
      if (out_values) export_dense(vals, out_values);
      export_dense(idx, out_indices);
    } else {
      auto iter = vbt::core::TensorIter::reduce_op(vals, base, std::span<const int64_t>(&rd, 1));
      if (dt == ScalarType::Float32)
        vbt::core::for_each_reduction_cpu(iter, kind == 0 ? &amax_f32 : &amin_f32, nullptr);
      else if (kind == 0)
        vbt::core::for_each_reduction_cpu(iter, &amax_i64, nullptr);
      else
        throw std::invalid_argument("amin int64 not wired in shim");
      export_dense(vals, out_values);
    }
  });
}

// op: "vt::add", "vt::mul", "vt::sub", "vt::div", "vt::eq" ... (binary) or
// "vt::relu", "vt::abs", "vt::neg", "vt::reciprocal" (unary; b ignored).
// out receives the dense broadcast result; out_sizes/out_ndim report its shape.
int vref_elementwise(const char* op, const void* a, int a_dtype, int a_ndim, const int64_t* a_sizes,
                     const int64_t* a_strides, const void* b, int b_dtype, int b_ndim,
                     const int64_t* b_sizes, const int64_t* b_strides, void* out,
                     int64_t* out_sizes, int* out_ndim) {
  return guarded([&] {
    ensure_registered();
    vbt::dispatch::BoxedStack s;
    s.push_back(wrap(a, a_dtype, a_ndim, a_sizes, a_strides));
    if (b) s.push_back(wrap(b, b_dtype, b_ndim, b_sizes, b_strides));
    vbt::dispatch::Dispatcher::instance().callBoxed(std::string(op), s);
    const TensorImpl& r = s.at(0);
    *out_ndim = static_cast<int>(r.sizes().size());
    for (std::size_t i = 0; i < r.sizes().size(); ++i) out_sizes[i] = r.sizes()[i];
    export_dense(r, out);
  });
}

// out[i, :] = self[idx[i], :]   through  indexing::index(self, {Tensor idx}).
// self is [V, D] (any supported dtype), idx int64 [N]; N*D <= 1e8 per call
// (indexing_advanced.cc:100-103) -- the caller chunks.
int vref_index_rows(const void* self, int dtype, int64_t V, int64_t D, int64_t s0, int64_t s1,
                    const int64_t* idx, int64_t N, void* out) {
  return guarded([&] {
    int64_t sz[2] = {V, D}, st[2] = {s0, s1};
    TensorImpl t = wrap(self, dtype, 2, sz, st);
    int64_t isz[1] = {N}, ist[1] = {1};
    TensorImpl it = wrap(idx, static_cast<int>(ScalarType::Int64), 1, isz, ist);
    vbt::core::indexing::IndexSpec spec;
    spec.items.emplace_back(it);
    TensorImpl r = vbt::core::indexing::index(t, spec);
    export_dense(r, out);
  });
}

// self[idx[i], :] (+)= value[i, :]  through indexing::index_put_.
int vref_index_put_rows(void* self, int dtype, int64_t V, int64_t D, const int64_t* idx, int64_t N,
                        const void* value, int accumulate) {
  return guarded([&] {
    int64_t sz[2] = {V, D}, st[2] = {D, 1};
    TensorImpl t = wrap(self, dtype, 2, sz, st);
    int64_t isz[1] = {N}, ist[1] = {1};
    TensorImpl it = wrap(idx, static_cast<int>(ScalarType::Int64), 1, isz, ist);
    int64_t vsz[2] = {N, D}, vst[2] = {D, 1};
    TensorImpl v = wrap(value, dtype, 2, vsz, vst);
    vbt::core::indexing::IndexSpec spec;
    spec.items.emplace_back(it);
    vbt::core::indexing::index_put_(t, spec, v, accumulate != 0);
  });
}

// 1-D forms (the shapes the reference's own unit tests use).
int vref_index_1d(const void* self, int dtype, int64_t n, const int64_t* idx, int64_t N,
                  void* out) {
  return guarded([&] {
    int64_t sz[1] = {n}, st[1] = {1};
    TensorImpl t = wrap(self, dtype, 1, sz, st);
    int64_t isz[1] = {N};
    TensorImpl it = wrap(idx, static_cast<int>(ScalarType::Int64), 1, isz, st);
    vbt::core::indexing::IndexSpec spec;
    spec.items.emplace_back(it);
    export_dense(vbt::core::indexing::index(t, spec), out);
  });
}
int vref_index_put_1d(void* self, int dtype, int64_t n, const int64_t* idx, int64_t N,
                      const void* value, int accumulate) {
  return guarded([&] {
    int64_t sz[1] = {n}, st[1] = {1};
    TensorImpl t = wrap(self, dtype, 1, sz, st);
    int64_t isz[1] = {N};
    TensorImpl it = wrap(idx, static_cast<int>(ScalarType::Int64), 1, isz, st);
    TensorImpl v = wrap(value, dtype, 1, isz, st);
    vbt::core::indexing::IndexSpec spec;
    spec.items.emplace_back(it);
    vbt::core::indexing::index_put_(t, spec, v, accumulate != 0);
  });
}

// out[i, :] = weight[idx[i], :]  through the boxed CPU "vt::embedding".
int vref_embedding(const float* weight, int64_t V, int64_t D, int64_t s0, int64_t s1,
                   const int64_t* idx, int64_t N, float* out) {
  return guarded([&] {
    ensure_registered();
    int64_t sz[2] = {V, D}, st[2] = {s0, s1};
    TensorImpl w = wrap(weight, static_cast<int>(ScalarType::Float32), 2, sz, st);
    int64_t isz[1] = {N}, ist[1] = {1};
    TensorImpl it = wrap(idx, static_cast<int>(ScalarType::Int64), 1, isz, ist);
    int64_t pad = -1;
    bool f = false;
    TensorImpl pad_t = wrap(&pad, static_cast<int>(ScalarType::Int64), 0, nullptr, nullptr);
    TensorImpl f1 = wrap(&f, static_cast<int>(ScalarType::Bool), 0, nullptr, nullptr);
    TensorImpl f2 = wrap(&f, static_cast<int>(ScalarType::Bool), 0, nullptr, nullptr);
    vbt::dispatch::BoxedStack s{w, it, pad_t, f1, f2};
    vbt::dispatch::Dispatcher::instance().callBoxed(std::string("vt::embedding"), s);
    export_dense(s.at(0), out);
  });
}

}  // extern "C"
