// Error plumbing and version query of the q4b200 C ABI.
#include <stdarg.h>
#include <string.h>

#include "q4_common.cuh"

namespace q4 {

char* err_buf() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return Q4_OK;
  return fail(Q4_E_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

int check_device() {
  static int ok[64] = {0};      // 0 unknown, 1 ok, -1 bad
  int dev = 0;
  if (int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
  if (dev >= 0 && dev < 64 && ok[dev] == 1) return Q4_OK;
  int major = 0, minor = 0;
  if (int e = check_cuda(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "device attribute")) return e;
  if (int e = check_cuda(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev), "device attribute")) return e;
  if (major != 10) return fail(Q4_E_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, major, minor);
  if (dev >= 0 && dev < 64) ok[dev] = 1;
  return Q4_OK;
}

}  // namespace q4

extern "C" int q4_version(void) { return Q4_VERSION; }
extern "C" const char* q4_last_error_string(void) { return q4::err_buf(); }
