// Error plumbing of the C ABI (int status + thread-local message) and the device check; linked into every
// library built from this directory.
#include <stdarg.h>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[1024] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  set_error("CUDA error %d (%s) at %s:%d in %s", (int)e, cudaGetErrorString(e), file, line, what);
  return B200_ERR_CUDA;
}

}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_last_error(void) { return g_err; }
int b200_abi_version(void) { return B200_ABI_VERSION; }

int b200_device_check(int device, int* sm_count) {
  cudaDeviceProp prop;
  B200_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
              prop.minor);
    return B200_ERR_UNSUPPORTED;
  }
  if (sm_count) *sm_count = prop.multiProcessorCount;
  return B200_OK;
}

}  // extern "C"
