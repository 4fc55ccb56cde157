// Split-KV decode whose scratch memory is part of the library image.
//
// Who this is for: a serving engine measures free HBM once, hands all of it to the KV cache and
// from then on must not call cudaMalloc (the memory is spoken for, and an allocation would also
// synchronise the device in the middle of a decode step).  Such a caller can still use the split
// decode through this entry point, because the partial results (normalised O and LSE of every
// split) land in a fixed array that every GPU loading the library holds until the process exits.
#include <cstdio>
#include <mutex>

#include "../../include/nvfp4_b200.h"
#include "nvfp4_kernels.h"

namespace {

constexpr size_t kStaticWorkspaceBytes = NVFP4_STATIC_WORKSPACE_BYTES;

// Device memory, one copy per GPU that loads the library.  In host code this name is only a
// handle for cudaGetSymbolAddress; it is never passed to a kernel as if it were an address.
static __device__ __align__(256) unsigned char g_split_workspace[kStaticWorkspaceBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_workspace_address[kMaxDevices] = {};
bool g_workspace_ready[kMaxDevices] = {};

// Resolves the array's device address for the CURRENT device, once per device.
cudaError_t workspace_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_workspace_ready[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_split_workspace);
    if (e != cudaSuccess) return e;
    g_workspace_address[dev] = ptr;
    g_workspace_ready[dev] = true;
  }
  *out = g_workspace_address[dev];
  return cudaSuccess;
}

thread_local char g_static_error[256] = "";

}  // namespace

extern "C" {

const char* nvfp4_decode_split_static_error(void) { return g_static_error; }

size_t nvfp4_static_workspace_bytes(void) { return kStaticWorkspaceBytes; }

int nvfp4_decode_split_static(const nvfp4_decode_args* args, void* stream) {
  g_static_error[0] = 0;
  // Set-up comes before every argument check.  Resolving the array's address the first time on
  // a device makes the CUDA runtime load the module that holds the array, and that takes the
  // array's bytes out of the device's free memory - once, not per call, and not through
  // cudaMalloc.  A caller that must know its free memory exactly (an engine about to size its
  // KV cache) therefore makes one call first - a call with args = NULL does the set-up and is
  // then refused - and every later call on that device leaves the free memory alone.
  void* workspace = nullptr;
  cudaError_t e = workspace_for_current_device(&workspace);
  if (e != cudaSuccess) {
    snprintf(g_static_error, sizeof(g_static_error), "decode_split_static: cudaGetSymbolAddress: %s",
             cudaGetErrorString(e));
    return NVFP4_ERR_CUDA;
  }
  if (!args) {
    snprintf(g_static_error, sizeof(g_static_error), "decode_split_static: null argument block");
    return NVFP4_ERR_INVALID;
  }
  if (args->num_splits < 2 || !args->out || args->o_partial || args->lse_partial) {
    snprintf(g_static_error, sizeof(g_static_error),
             "decode_split_static: needs num_splits >= 2, an output buffer and no caller-owned partials");
    return NVFP4_ERR_INVALID;
  }
  const size_t need = nvfp4_decode_workspace_bytes(args->rows, args->heads_q, args->num_splits);
  if (need > kStaticWorkspaceBytes) {
    snprintf(g_static_error, sizeof(g_static_error),
             "decode_split_static: %d splits x %d rows x %d heads need %zu bytes of partials, the built-in "
             "workspace holds %zu; use nvfp4_decode with a caller-owned workspace",
             args->num_splits, args->rows, args->heads_q, need, kStaticWorkspaceBytes);
    return NVFP4_ERR_INVALID;
  }
  nvfp4_decode_args with_ws = *args;
  with_ws.workspace = workspace;
  with_ws.workspace_bytes = kStaticWorkspaceBytes;
  const int rc = nvfp4_decode(&with_ws, stream);
  if (rc != NVFP4_OK) snprintf(g_static_error, sizeof(g_static_error), "%s", nvfp4_last_error());
  return rc;
}

}  // extern "C"
