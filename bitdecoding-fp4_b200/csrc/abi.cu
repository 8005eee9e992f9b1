// Library-level entry points: version, status text, device check.
#include <cstdio>
#include <cstring>

#include "host.h"

namespace bdfp4 {

static thread_local char g_last_error[256] = "";

int cuda_status(cudaError_t error) {
  if (error == cudaSuccess) return BDFP4_OK;
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", cudaGetErrorName(error), cudaGetErrorString(error));
  return BDFP4_E_CUDA;
}

}  // namespace bdfp4

extern "C" int bdfp4_version(void) { return 100; }

extern "C" const char* bdfp4_status_string(int status) {
  switch (status) {
    case BDFP4_OK: return "ok";
    case BDFP4_E_ARG: return "argument violates the documented contract";
    case BDFP4_E_UNSUPPORTED: return "request is valid but this build has no kernel for it";
    case BDFP4_E_CUDA: return "a CUDA call failed";
    case BDFP4_E_DEVICE: return "the current device is not an sm_100-family GPU";
    case BDFP4_E_TOO_LARGE: return "the request exceeds a fixed-capacity buffer of the library";
    default: return "unknown status";
  }
}

extern "C" const char* bdfp4_last_cuda_error(void) { return bdfp4::g_last_error; }

extern "C" int bdfp4_check_device(void) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return bdfp4::cuda_status(e);
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) return bdfp4::cuda_status(e);
  return major == 10 ? BDFP4_OK : BDFP4_E_DEVICE;
}
