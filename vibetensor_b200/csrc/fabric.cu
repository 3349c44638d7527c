// vt::fabric_add / vt::fabric_mul: a binary op whose operands live on two GPUs of one process.
//
// Replaces fabric_addmul_impl and its kernels (src/vbt/cuda/fabric_elementwise.cu:122-162,
// :478-593, :820-1042) with the contract of its entry points
// vbt_cuda_fabric_{add,mul}_impl(a, b, compute_device, require_fabric, use_copy_fallback)
// (:1052-1115):
//   * equal shapes and dtypes, CUDA operands, else a "[Fabric] ..." error;
//   * both operands on one device: the ordinary op on that device;
//   * two devices: compute_device must be one of them and owns the output.  When that device can
//     open the other's memory, the elementwise kernel reads the remote operand in place with plain
//     loads over NVLink (no staging copy, no second pass) -- the "fabric" mode.  When it cannot
//     (or the caller asks for the dry-run behaviour), and the policy allows it, the remote
//     operand is first copied into caller-provided local scratch with cudaMemcpyPeerAsync and
//     the op then runs locally -- the copy fallback (:281-367, decision :603-663).  Otherwise
//     the call fails with the reference's message.
// No cluster-multicast load, and no library kernel, ever sees the peer pointer: only this
// library's own elementwise kernels dereference it.
#include "common.cuh"

namespace vb {
namespace {

const char* fabric_name(int op) {
  return op == VBT_B200_B_ADD ? "vt::fabric_add" : (op == VBT_B200_B_MUL ? "vt::fabric_mul" : "vt::fabric_binary");
}

// device that owns a pointer, or -1
int owner_device(const void* p) {
  cudaPointerAttributes attr{};
  if (p && cudaPointerGetAttributes(&attr, p) == cudaSuccess &&
      (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged))
    return attr.device;
  cudaGetLastError();
  return -1;
}

}  // namespace
}  // namespace vb

extern "C" vbt_b200_status vbt_b200_fabric_binary(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                                  const vbt_b200_tensor* b, int32_t compute_device,
                                                  int32_t require_fabric, int32_t use_copy_fallback, void* scratch,
                                                  size_t scratch_bytes, int32_t* mode_out, void* stream) {
  using namespace vb;
  const std::string name = fabric_name(op);
  if (mode_out) *mode_out = 0;
  VB_TRY(validate_data(out, name.c_str()));
  VB_TRY(validate_data(a, name.c_str()));
  VB_TRY(validate_data(b, name.c_str()));
  bool same_shape = a->ndim == b->ndim;
  for (int d = 0; same_shape && d < a->ndim; ++d) same_shape = a->sizes[d] == b->sizes[d];
  VB_REQUIRE(same_shape, VBT_B200_RUNTIME_ERROR, "[Fabric] " + name + ": requires equal shapes");
  VB_REQUIRE(a->dtype == b->dtype, VBT_B200_RUNTIME_ERROR, "[Fabric] " + name + ": requires equal dtypes");
  if (numel(*a) == 0) return vbt_b200_binary(op, out, a, b, stream);
  const int da = owner_device(a->data), db = owner_device(b->data), dout = owner_device(out->data);
  VB_REQUIRE(da >= 0 && db >= 0 && dout >= 0, VBT_B200_RUNTIME_ERROR, "[Fabric] " + name + ": expects CUDA tensors");
  if (da == db) {  // single-device case: the ordinary op
    VB_REQUIRE(dout == da, VBT_B200_RUNTIME_ERROR, "[Fabric] " + name + ": the output must live on the operands' device");
    VB_TRY(vbt_b200_binary(op, out, a, b, stream));
    if (mode_out) *mode_out = VBT_B200_FK_LOCAL;
    launch_info_ref().family = VBT_B200_FAMILY_FABRIC;
    launch_info_ref().kernel = VBT_B200_FK_LOCAL;
    return VBT_B200_OK;
  }
  VB_REQUIRE(compute_device == da || compute_device == db, VBT_B200_RUNTIME_ERROR,
             "[Fabric] " + name + ": compute_device must be the device of one of the operands");
  VB_REQUIRE(dout == compute_device, VBT_B200_RUNTIME_ERROR,
             "[Fabric] " + name + ": the output must live on compute_device");
  const int primary = compute_device, other = compute_device == da ? db : da;
  const vbt_b200_tensor* remote = compute_device == da ? b : a;
  int can = 0;
  VB_CUDA(cudaDeviceCanAccessPeer(&can, primary, other));
  const bool dry_run = use_copy_fallback == 2 && !require_fabric;  // the reference's DryRun mode: copy even when P2P exists
  if (can && !dry_run) {
    VB_TRY(vbt_b200_enable_peer_access(primary, other));
    VB_TRY(vbt_b200_binary(op, out, a, b, stream));  // the remote operand is read in place over NVLink
    if (mode_out) *mode_out = VBT_B200_FK_PEER_LOAD;
    launch_info_ref().family = VBT_B200_FAMILY_FABRIC;
    launch_info_ref().kernel = VBT_B200_FK_PEER_LOAD;
    return VBT_B200_OK;
  }
  if (require_fabric || !use_copy_fallback)
    return fail(VBT_B200_RUNTIME_ERROR, "[Fabric] " + name +
                                            ": peer access not available for the selected device pair (primary=" +
                                            std::to_string(primary) + ", remote=" + std::to_string(other) + ")");
  // copy fallback: bring the remote operand into local scratch, then compute locally
  VB_REQUIRE(is_dense_row_major(*remote), VBT_B200_RUNTIME_ERROR,
             "[Fabric] " + name + ": the copy fallback needs a contiguous remote operand");
  const size_t bytes = static_cast<size_t>(numel(*remote)) * itemsize(remote->dtype);
  VB_ARG(scratch != nullptr && scratch_bytes >= bytes && owner_device(scratch) == primary,
         "[Fabric] " + name + ": the copy fallback needs numel * itemsize bytes of scratch on compute_device");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    DeviceScope scope(out->data);
    VB_CUDA(cudaMemcpyPeerAsync(scratch, primary, remote->data, other, bytes, s));
  }
  vbt_b200_tensor local = *remote;
  local.data = scratch;
  VB_TRY(vbt_b200_binary(op, out, compute_device == da ? a : &local, compute_device == da ? &local : b, stream));
  if (mode_out) *mode_out = VBT_B200_FK_COPY_FALLBACK;
  launch_info_ref().family = VBT_B200_FAMILY_FABRIC;
  launch_info_ref().kernel = VBT_B200_FK_COPY_FALLBACK;
  launch_info_ref().launches += 1;
  return VBT_B200_OK;
}
