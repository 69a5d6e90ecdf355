// Library-level state: last error text, device properties.
#include "common.cuh"
#include <cstdarg>
#include <cstring>

static thread_local char g_last_error[512] = "";

int mtb_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int mtb_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int mtb_opt_in_smem(const void* kernel, int bytes, unsigned long long* done_mask) {
  int dev = 0;
  MTB_CUDA(cudaGetDevice(&dev));
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && ((__atomic_load_n(done_mask, __ATOMIC_ACQUIRE) >> dev) & 1ull)) return MTB_OK;
  MTB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (tracked) __atomic_fetch_or(done_mask, 1ull << dev, __ATOMIC_RELEASE);
  return MTB_OK;
}

namespace {
struct Lanes {
  cudaStream_t stream[kMaxLanes - 1];
  cudaEvent_t fork, join[kMaxLanes - 1];
  bool made;
};
Lanes g_lanes[64];
}  // namespace

int mtb_fork_lanes(cudaStream_t main, int lanes, cudaStream_t* out) {
  int dev = 0;
  MTB_CUDA(cudaGetDevice(&dev));
  MTB_REQUIRE(dev >= 0 && dev < 64 && lanes >= 1 && lanes <= kMaxLanes, "mtb_fork_lanes: device %d, %d lanes", dev, lanes);
  Lanes& l = g_lanes[dev];
  if (!l.made) {
    for (int i = 0; i < kMaxLanes - 1; ++i) {
      MTB_CUDA(cudaStreamCreateWithFlags(&l.stream[i], cudaStreamNonBlocking));
      MTB_CUDA(cudaEventCreateWithFlags(&l.join[i], cudaEventDisableTiming));
    }
    MTB_CUDA(cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming));
    l.made = true;
  }
  out[0] = main;
  if (lanes > 1) MTB_CUDA(cudaEventRecord(l.fork, main));
  for (int i = 1; i < lanes; ++i) {
    MTB_CUDA(cudaStreamWaitEvent(l.stream[i - 1], l.fork, 0));
    out[i] = l.stream[i - 1];
  }
  return MTB_OK;
}

int mtb_join_lanes(cudaStream_t main, int lanes) {
  int dev = 0;
  MTB_CUDA(cudaGetDevice(&dev));
  MTB_REQUIRE(dev >= 0 && dev < 64 && g_lanes[dev].made, "mtb_join_lanes without mtb_fork_lanes");
  Lanes& l = g_lanes[dev];
  for (int i = 1; i < lanes; ++i) {
    MTB_CUDA(cudaEventRecord(l.join[i - 1], l.stream[i - 1]));
    MTB_CUDA(cudaStreamWaitEvent(main, l.join[i - 1], 0));
  }
  return MTB_OK;
}

MTB_API const char* mtb_last_error() { return g_last_error; }

MTB_API int mtb_version() { return 1; }

// Returns MTB_OK when the current device can run this library (compute capability 10.x).
MTB_API int mtb_device_check() {
  int dev = 0, major = 0, minor = 0;
  MTB_CUDA(cudaGetDevice(&dev));
  MTB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  MTB_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
  if (major != 10) return mtb_fail(MTB_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, major, minor);
  return MTB_OK;
}
