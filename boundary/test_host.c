/*
 * TEST DOUBLE of the VibeTensor plugin host (not part of the product).
 *
 * Stands where src/vbt/dispatch/plugin_loader.cc stands for a real plugin: fills a
 * `struct vbt_host_api` (include/vbt/plugin/vbt_plugin.h), dlopens a plugin, checks its ABI
 * version the way the loader does (major equal, plugin minor <= host minor, :36-41), calls
 * vbt_plugin_init, and records what the plugin registers.  Tensors are plain descriptors over
 * device (or, for host-only tests, fake) pointers supplied by the test; outputs come from an
 * allocator callback the test installs (it hands out torch memory), are tracked per call, and
 * are dropped when a kernel fails -- the loader's AllocTracker behaviour
 * (plugin_loader.cc:1097-1103).  Like the real host it ignores registrations for "vt::add"
 * (:1183-1185), returns NULL from tensor_mutable_data for inputs (:1388-1395) and rejects ops
 * it has no schema for.
 */
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "vbt/plugin/vbt_plugin.h"

#define TH_EXPORT __attribute__((visibility("default")))
#define TH_MAX_KERNELS 512
#define TH_MAX_NDIM 25

struct vt_tensor__ {
  void* data;
  DLDataType dtype;
  DLDevice device;
  int32_t ndim;
  int64_t sizes[TH_MAX_NDIM];
  int64_t strides[TH_MAX_NDIM];
  int is_output;  /* created by tensor_new_dense_like during a kernel call */
};

typedef void* (*th_alloc_fn)(size_t bytes, int32_t device);

struct kernel_entry {
  char name[96];
  int arity; /* 2 = vt_kernel2_fn, -1 = boxed */
  vt_kernel2_fn k2;
  vt_kernel_boxed_fn boxed;
};

static struct kernel_entry g_kernels[TH_MAX_KERNELS];
static int g_nkernels;
static int g_ignored_add;
static char g_schemas[TH_MAX_KERNELS][96];
static int g_nschemas;
static int g_accept_all = 1; /* no schema list installed: every op name is defined */
static __thread char tl_err[512];
static th_alloc_fn g_alloc;
static vt_tensor g_live_outputs[64];
static int g_nlive;
static void* g_plugin;
static vt_stream g_stream;

/* ---- host API implementation ---------------------------------------------------------- */
static void host_set_last_error(const char* msg) {
  snprintf(tl_err, sizeof(tl_err), "%s", msg ? msg : "");
}
static int has_schema(const char* fq) {
  if (g_accept_all) return 1;
  for (int i = 0; i < g_nschemas; ++i)
    if (strcmp(g_schemas[i], fq) == 0) return 1;
  return 0;
}
static vt_status add_kernel(const char* fq, vt_dispatch_key key, vt_kernel2_fn k2, vt_kernel_boxed_fn boxed) {
  tl_err[0] = 0;
  if (!fq) { host_set_last_error("invalid argument: fqname is null"); return VT_STATUS_INVALID_ARG; }
  if (!*fq) { host_set_last_error("invalid argument: fqname is empty"); return VT_STATUS_INVALID_ARG; }
  if (!k2 && !boxed) { host_set_last_error("null kernel"); return VT_STATUS_INVALID_ARG; }
  if (key != kDLCPU && key != kDLCUDA) { host_set_last_error("unsupported dispatch key"); return VT_STATUS_UNSUPPORTED; }
  if (strcmp(fq, "vt::add") == 0) { ++g_ignored_add; return VT_STATUS_OK; }
  if (!has_schema(fq)) {
    snprintf(tl_err, sizeof(tl_err), "undefined op in VBT_IMPL_CUDA: %s", fq);
    return VT_STATUS_INVALID_ARG;
  }
  for (int i = 0; i < g_nkernels; ++i)
    if (strcmp(g_kernels[i].name, fq) == 0) { /* replace, as replaceCudaKernelFunction does */
      g_kernels[i].k2 = k2; g_kernels[i].boxed = boxed; g_kernels[i].arity = k2 ? 2 : -1;
      return VT_STATUS_OK;
    }
  if (g_nkernels == TH_MAX_KERNELS) { host_set_last_error("too many kernels"); return VT_STATUS_NOMEM; }
  struct kernel_entry* e = &g_kernels[g_nkernels++];
  snprintf(e->name, sizeof(e->name), "%s", fq);
  e->arity = k2 ? 2 : -1;
  e->k2 = k2;
  e->boxed = boxed;
  return VT_STATUS_OK;
}
static vt_status host_register_kernel2(const char* fq, vt_dispatch_key key, vt_kernel2_fn fn) {
  return add_kernel(fq, key, fn, NULL);
}
static vt_status host_register_kernel_boxed(const char* fq, vt_dispatch_key key, vt_kernel_boxed_fn fn) {
  return add_kernel(fq, key, NULL, fn);
}
static vt_status host_register_cuda_kernel2(const char* fq, vt_kernel2_fn fn) { return add_kernel(fq, kDLCUDA, fn, NULL); }
static vt_status host_register_library(const char* ns) { (void)ns; return VT_STATUS_OK; }
static vt_status host_def(const char* def_string) { (void)def_string; return VT_STATUS_OK; }

static int64_t host_numel(vt_tensor t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->sizes[i];
  return n;
}
static DLDataType host_dtype(vt_tensor t) { return t->dtype; }
static DLDevice host_device(vt_tensor t) { return t->device; }
static size_t host_ndim(vt_tensor t) { return (size_t)t->ndim; }
static const int64_t* host_sizes(vt_tensor t) { return t->ndim ? t->sizes : NULL; }
static const int64_t* host_strides(vt_tensor t) { return t->ndim ? t->strides : NULL; }
static int64_t host_storage_offset(vt_tensor t) { (void)t; return 0; }
static size_t host_itemsize(vt_tensor t) { return (size_t)(t->dtype.bits * t->dtype.lanes + 7) / 8; }
static const void* host_data(vt_tensor t) { return t->data; }
static void* host_mutable_data(vt_tensor t) { return t->is_output ? t->data : NULL; }
static int host_is_contiguous(vt_tensor t) {
  int64_t expect = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->sizes[i] != 1 && t->strides[i] != expect) return 0;
    expect *= t->sizes[i];
  }
  return 1;
}
static vt_status host_new_dense_like(vt_tensor like, vt_tensor* out) {
  if (!like || !out) { host_set_last_error("null argument"); return VT_STATUS_INVALID_ARG; }
  if (g_nlive == 64) { host_set_last_error("too many live outputs"); return VT_STATUS_NOMEM; }
  vt_tensor t = (vt_tensor)calloc(1, sizeof(*t));
  if (!t) return VT_STATUS_NOMEM;
  *t = *like;
  int64_t stride = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    t->strides[i] = stride;
    stride *= t->sizes[i];
  }
  t->is_output = 1;
  const size_t bytes = (size_t)host_numel(t) * host_itemsize(t);
  t->data = NULL;
  if (bytes) {
    t->data = g_alloc ? g_alloc(bytes, t->device.device_id) : NULL;
    if (!t->data) {
      free(t);
      host_set_last_error("allocation failed");
      return VT_STATUS_NOMEM;
    }
  }
  g_live_outputs[g_nlive++] = t;
  *out = t;
  return VT_STATUS_OK;
}
static vt_stream host_current_stream(int32_t device_index) { (void)device_index; return g_stream; }

static struct vbt_host_api g_host;

static void fill_host(uint32_t minor) {
  memset(&g_host, 0, sizeof(g_host));
  g_host.host_abi_major = VBT_PLUGIN_ABI_VERSION_MAJOR;
  g_host.host_abi_minor = minor;
  g_host.register_library = host_register_library;
  g_host.def = host_def;
  g_host.tensor_numel = host_numel;
  g_host.tensor_dtype = host_dtype;
  g_host.tensor_device = host_device;
  g_host.tensor_ndim = host_ndim;
  g_host.tensor_sizes = host_sizes;
  g_host.tensor_strides = host_strides;
  g_host.tensor_storage_offset = host_storage_offset;
  g_host.tensor_itemsize = host_itemsize;
  g_host.tensor_data = host_data;
  g_host.tensor_mutable_data = host_mutable_data;
  g_host.tensor_is_contiguous = host_is_contiguous;
  g_host.tensor_new_dense_like = host_new_dense_like;
  g_host.set_last_error = host_set_last_error;
  g_host.register_cuda_kernel2 = host_register_cuda_kernel2;
  g_host.current_cuda_stream = host_current_stream;
  g_host.register_kernel_boxed = host_register_kernel_boxed;
  g_host.register_kernel2 = host_register_kernel2;
  /* the TensorIterator helpers and set_device_policy stay NULL: this path does not use them */
}

/* ---- what the tests drive -------------------------------------------------------------- */
TH_EXPORT void th_set_allocator(th_alloc_fn fn) { g_alloc = fn; }
TH_EXPORT void th_set_stream(uint64_t s) { g_stream = s; }
/* Restrict the ops the host "defines"; n == 0 goes back to accepting every name. */
TH_EXPORT void th_set_schemas(const char* const* names, int n) {
  g_accept_all = n == 0;
  g_nschemas = 0;
  for (int i = 0; i < n && i < TH_MAX_KERNELS; ++i) snprintf(g_schemas[g_nschemas++], 96, "%s", names[i]);
}
TH_EXPORT const char* th_last_error(void) { return tl_err; }

/* Loads the plugin as the loader does.  Returns the vt_status of the load; *abi receives the
 * plugin's reported ABI word, name_out (may be NULL) the plugin's display name. */
TH_EXPORT int th_load_plugin(const char* path, uint32_t host_minor, uint32_t* abi, const char** name_out) {
  g_nkernels = 0;
  g_ignored_add = 0;
  tl_err[0] = 0;
  if (g_plugin) { dlclose(g_plugin); g_plugin = NULL; }
  g_plugin = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!g_plugin) {
    snprintf(tl_err, sizeof(tl_err), "dlopen: %s", dlerror());
    return VT_STATUS_NOT_FOUND;
  }
  uint32_t (*get_abi)(void) = (uint32_t (*)(void))dlsym(g_plugin, "vbt_plugin_get_abi_version");
  vt_status (*init)(const struct vbt_host_api*, struct vbt_plugin_api*) =
      (vt_status (*)(const struct vbt_host_api*, struct vbt_plugin_api*))dlsym(g_plugin, "vbt_plugin_init");
  if (!get_abi || !init) {
    host_set_last_error("plugin lacks vbt_plugin_get_abi_version / vbt_plugin_init");
    return VT_STATUS_NOT_FOUND;
  }
  const uint32_t v = get_abi();
  if (abi) *abi = v;
  if ((v >> 16) != VBT_PLUGIN_ABI_VERSION_MAJOR || (v & 0xffffu) > host_minor) {
    host_set_last_error("ABI mismatch");
    return VT_STATUS_ABI_MISMATCH;
  }
  fill_host(host_minor);
  struct vbt_plugin_api api;
  memset(&api, 0, sizeof(api));
  const vt_status st = init(&g_host, &api);
  if (st == VT_STATUS_OK && name_out) *name_out = api.name;
  if (st == VT_STATUS_OK && api.abi_version != v) {
    host_set_last_error("plugin_api.abi_version differs from vbt_plugin_get_abi_version()");
    return VT_STATUS_ABI_MISMATCH;
  }
  return st;
}
TH_EXPORT int th_num_kernels(void) { return g_nkernels; }
TH_EXPORT int th_ignored_add(void) { return g_ignored_add; }
TH_EXPORT const char* th_kernel_name(int i) { return (i >= 0 && i < g_nkernels) ? g_kernels[i].name : NULL; }
TH_EXPORT int th_kernel_arity(int i) { return (i >= 0 && i < g_nkernels) ? g_kernels[i].arity : 0; }
TH_EXPORT void* th_plugin_symbol(const char* name) { return g_plugin ? dlsym(g_plugin, name) : NULL; }

/* dtype: DLPack (code, bits); device_type kDLCUDA = 2, kDLCPU = 1 */
TH_EXPORT vt_tensor th_make_tensor(void* data, int code, int bits, int device_type, int device_id, int ndim,
                                   const int64_t* sizes, const int64_t* strides) {
  if (ndim < 0 || ndim > TH_MAX_NDIM) return NULL;
  vt_tensor t = (vt_tensor)calloc(1, sizeof(*t));
  if (!t) return NULL;
  t->data = data;
  t->dtype.code = (uint8_t)code;
  t->dtype.bits = (uint8_t)bits;
  t->dtype.lanes = 1;
  t->device.device_type = (DLDeviceType)device_type;
  t->device.device_id = device_id;
  t->ndim = ndim;
  for (int i = 0; i < ndim; ++i) {
    t->sizes[i] = sizes[i];
    t->strides[i] = strides[i];
  }
  return t;
}
TH_EXPORT void th_free_tensor(vt_tensor t) { free(t); }
TH_EXPORT void* th_tensor_data(vt_tensor t) { return t ? t->data : NULL; }
TH_EXPORT int th_tensor_ndim(vt_tensor t) { return t ? t->ndim : -1; }
TH_EXPORT int64_t th_tensor_size(vt_tensor t, int i) { return t->sizes[i]; }

/* Calls a registered kernel the way the dispatcher trampoline does.  On a non-OK status the
 * outputs the kernel created are dropped and *out is NULL. */
TH_EXPORT int th_call(const char* fq, const vt_tensor* args, int nargs, vt_tensor* out) {
  tl_err[0] = 0;
  *out = NULL;
  g_nlive = 0;
  for (int i = 0; i < g_nkernels; ++i) {
    if (strcmp(g_kernels[i].name, fq) != 0) continue;
    vt_status st;
    if (g_kernels[i].arity == 2) {
      if (nargs != 2) { host_set_last_error("arity mismatch"); return VT_STATUS_INVALID_ARG; }
      st = g_kernels[i].k2(g_stream, args[0], args[1], out);
    } else {
      st = g_kernels[i].boxed(g_stream, args, (size_t)nargs, out);
    }
    if (st != VT_STATUS_OK) {
      for (int k = 0; k < g_nlive; ++k) free(g_live_outputs[k]);
      *out = NULL;
    } else {
      for (int k = 0; k < g_nlive; ++k)
        if (g_live_outputs[k] != *out) free(g_live_outputs[k]);
    }
    g_nlive = 0;
    return st;
  }
  host_set_last_error("no such kernel");
  return VT_STATUS_NOT_FOUND;
}
