// Forward with library-owned scratch memory: one entry point for callers that cannot
// hand over a workspace and must not allocate.
//
// Some hosts give a plugin nothing but input and output buffers and a stream: a serving
// runtime whose per-request hook has no workspace argument, or a process whose framework
// reserved the whole device up front, so that a cudaMalloc issued from inside a library
// call fails.  For them the scratch that dcn_fwd normally receives from its caller (status
// word, swizzled weight image, channels-last copy of the input) lives in a fixed array that
// is part of this library's device image; every GPU that loads the library holds those
// DCN_STATIC_SCRATCH_BYTES until the process exits.
//
// The array is shared by every call on a device and keeps whatever the previous call left
// in it.  Nothing in it has to start at zero except the status word, which the first
// kernel of every call clears; the weight image and the input copy are rewritten in full
// before they are read.  Two calls that overlap on the same GPU (different streams or
// threads) both write the array and race: serialise them.
#include <cstdio>
#include <mutex>

#include "dcn_internal.cuh"

namespace {

// In host code this name is only a handle for the runtime, not a device address: passing it
// to a kernel as is would fault (or, where the GPU can reach host memory, quietly use the
// wrong bytes).  Host code below asks the runtime for the real address, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[DCN_STATIC_SCRATCH_BYTES];

std::mutex g_static_mu;
void *g_static_ptr[64] = {nullptr};

}  // namespace

extern "C" int dcn_fwd_static_scratch(const DcnFwdParams *p, void *stream, void **scratch) {
  if (!p) return dcn::set_error(DCN_ERR_ARG, "params is NULL");
  size_t need = 0;
  const int rc = dcn_fwd_workspace_bytes(p, &need);
  if (rc) return rc;  // dcn_last_error() already says why
  if (need > (size_t)DCN_STATIC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "this problem needs %zu bytes of scratch; the built-in scratch array holds %zu "
             "(use dcn_fwd with a caller-provided workspace)",
             need, (size_t)DCN_STATIC_SCRATCH_BYTES);
    return dcn::set_error(DCN_ERR_WORKSPACE, msg);
  }
  if (p->device < 0 || p->device >= 64)
    return dcn::set_error(DCN_ERR_ARG, "device ordinal out of range");
  void *ptr = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    ptr = g_static_ptr[p->device];
    if (!ptr) {
      // Set-up, once per device and with that device current: resolve the array's address.
      // (the caller's current device is put back afterwards)
      int prev = -1;
      cudaError_t e = cudaGetDevice(&prev);
      if (e == cudaSuccess && prev != p->device) e = cudaSetDevice(p->device);
      if (e == cudaSuccess) e = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (prev >= 0 && prev != p->device) cudaSetDevice(prev);
      if (e != cudaSuccess || !ptr) {
        char msg[256];
        snprintf(msg, sizeof(msg), "cannot resolve the built-in scratch array on device %d: %s",
                 p->device, cudaGetErrorString(e));
        cudaGetLastError();
        return dcn::set_error(DCN_ERR_DEVICE, msg);
      }
      g_static_ptr[p->device] = ptr;
    }
  }
  if (scratch) *scratch = ptr;
  return dcn_fwd(p, ptr, (size_t)DCN_STATIC_SCRATCH_BYTES, stream);
}
