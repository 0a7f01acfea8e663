// Status strings, version and the device gate of the C ABI.
#include "common.cuh"

namespace tsb {
int g_last_cuda_error = 0;
int g_pdl = 0;

int check_device_cached() {
  // Cached per device ordinal: 0 = unknown, 1 = ok, 2 = wrong architecture.
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TSB200_ERR_CUDA;
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (cache[dev] == 0) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess)
      return TSB200_ERR_CUDA;
    cache[dev] = (major == 10 && minor == 0) ? 1 : 2;
  }
  return cache[dev] == 1 ? TSB200_OK : TSB200_ERR_DEVICE;
}
}  // namespace tsb

extern "C" {

const char* tsb200_strerror(int status) {
  switch (status) {
    case TSB200_OK: return "ok";
    case TSB200_ERR_ARG: return "invalid argument (null/misaligned pointer or bad size)";
    case TSB200_ERR_UNSUPPORTED: return "unsupported shape, dtype or format";
    case TSB200_ERR_CUDA: return "CUDA runtime error (see tsb200_last_cuda_error)";
    case TSB200_ERR_WORKSPACE: return "workspace too small";
    case TSB200_ERR_DEVICE: return "device is not compute capability 10.0 (sm_100a only, no fallback)";
    case TSB200_ERR_TIMEOUT: return "bounded device-side wait timed out";
    default: return "unknown status";
  }
}

int tsb200_version(void) { return 100; }
int tsb200_last_cuda_error(void) { return tsb::g_last_cuda_error; }
int tsb200_check_device(void) { return tsb::check_device_cached(); }
int tsb200_set_pdl(int enabled) {
  const int old = tsb::g_pdl;
  tsb::g_pdl = enabled ? 1 : 0;
  return old;
}

}  // extern "C"
