// Library-level plumbing of the C ABI: error reporting, device checks, the device status word.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "lq_common.cuh"

namespace lq {

static thread_local char g_last_cuda_error[256] = "";

// Written by bounded device-side waits that give up (value = site code); read by lq_poll_status.
__device__ int g_status_word = 0;

void record_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%d)", where,
           cudaGetErrorString(e), static_cast<int>(e));
}

int check_launch(const char* where) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    record_cuda_error(e, where);
    return LQ_ERR_CUDA;
  }
  return LQ_OK;
}

static constexpr int kMaxDevices = 64;
static int g_sm_count[kMaxDevices];
static int g_cc_major[kMaxDevices];
static int* g_status_ptr[kMaxDevices];
static std::once_flag g_dev_once[kMaxDevices];

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  std::call_once(g_dev_once[dev], [dev]() {
    cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&g_cc_major[dev], cudaDevAttrComputeCapabilityMajor, dev);
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) == cudaSuccess) g_status_ptr[dev] = static_cast<int*>(p);
  });
  return dev;
}

int sm_count() {
  int dev = current_device();
  return dev < 0 || g_sm_count[dev] <= 0 ? 148 : g_sm_count[dev];
}

bool pdl_enabled() {
  static const bool on = []() {
    const char* e = getenv("LIQUIDGEMM_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

int* status_word() {
  int dev = current_device();
  return dev < 0 ? nullptr : g_status_ptr[dev];
}

}  // namespace lq

extern "C" {

int lq_abi_version(void) { return 1; }

const char* lq_error_string(int code) {
  switch (code) {
    case LQ_OK: return "ok";
    case LQ_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown dtype code)";
    case LQ_ERR_SHAPE: return "shape precondition violated";
    case LQ_ERR_WORKSPACE: return "workspace missing or too small";
    case LQ_ERR_CUDA: return "CUDA call failed";
    case LQ_ERR_DEVICE: return "current device is not compute capability 10.x";
    case LQ_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    default: return "unknown error code";
  }
}

const char* lq_last_cuda_error(void) { return lq::g_last_cuda_error; }

int lq_check_device(void) {
  int dev = lq::current_device();
  if (dev < 0) return LQ_ERR_CUDA;
  return lq::g_cc_major[dev] == 10 ? LQ_OK : LQ_ERR_DEVICE;
}

int lq_poll_status(void* stream) {
  int* p = lq::status_word();
  if (!p) return LQ_ERR_CUDA;
  int host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, p, sizeof(int), cudaMemcpyDeviceToHost, lq::as_stream(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(lq::as_stream(stream));
  if (e != cudaSuccess) {
    lq::record_cuda_error(e, "lq_poll_status");
    return LQ_ERR_CUDA;
  }
  if (host != 0) {
    cudaMemsetAsync(p, 0, sizeof(int), lq::as_stream(stream));
    snprintf(lq::g_last_cuda_error, sizeof(lq::g_last_cuda_error), "device wait timed out at site %d", host);
    return LQ_ERR_TIMEOUT;
  }
  return LQ_OK;
}

}  // extern "C"
