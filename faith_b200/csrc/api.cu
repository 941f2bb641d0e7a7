// Status strings, error bookkeeping and the per-device property cache of libfaith_b200.
#include <mutex>

#include "common.cuh"

namespace fb {

static thread_local int t_last_cuda_error = 0;
void set_last_cuda_error(int e) { t_last_cuda_error = e; }

namespace {
constexpr int kMaxDevices = 64;
DeviceInfo g_info[kMaxDevices];
std::once_flag g_once[kMaxDevices];
}  // namespace

const DeviceInfo& device_info() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  std::call_once(g_once[dev], [dev]() {
    int sms = 148, smem = 227 * 1024;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    g_info[dev].sms = sms;
    g_info[dev].smem_optin = smem;
  });
  return g_info[dev];
}

}  // namespace fb

extern "C" const char* fb_status_string(int status) {
  switch (status) {
    case FB_OK: return "ok";
    case FB_ERR_ARG: return "invalid argument (null pointer, negative size or unknown enum value)";
    case FB_ERR_SHAPE: return "unsupported shape";
    case FB_ERR_ALIGN: return "pointer not 16-byte aligned";
    case FB_ERR_CUDA: return "CUDA runtime error (see fb_last_cuda_error)";
    case FB_ERR_WORKSPACE: return "workspace too small";
    default: return "unknown status";
  }
}

extern "C" int fb_last_cuda_error(void) { return fb::t_last_cuda_error; }
extern "C" int fb_version(void) { return 100; }
