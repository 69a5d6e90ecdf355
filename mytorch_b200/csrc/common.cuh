// Shared helpers for the sm_100a kernel library: error reporting, launch checks, grid sizing.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define MTB_API extern "C" __attribute__((visibility("default")))

enum MtbStatus {
  MTB_OK = 0,
  MTB_ERR_INVALID = 1,      // bad argument (null pointer, negative size, unsupported shape)
  MTB_ERR_CUDA = 2,         // a CUDA runtime / driver call failed
  MTB_ERR_UNSUPPORTED = 3,  // shape not covered by the requested kernel family
  MTB_ERR_WORKSPACE = 4,    // caller's scratch buffer is too small
  MTB_ERR_DEVICE = 5,       // a kernel reported a device-side problem (bounded wait ran out)
};

int mtb_fail(int code, const char* fmt, ...);
int mtb_sm_count();
// Opt a kernel in to `bytes` of dynamic shared memory on the CURRENT device.  The attribute is kept
// per device, so `done_mask` (one per kernel, zero-initialised) remembers the ordinals already set.
int mtb_opt_in_smem(const void* kernel, int bytes, unsigned long long* done_mask);

// Lanes: up to three auxiliary streams per device for an entry point that enqueues several launches which
// do not depend on one another (and each fill only part of the GPU).  mtb_fork_lanes makes lanes 1..n-1 wait
// for everything enqueued on `main` so far and returns their streams (lane 0 is `main` itself);
// mtb_join_lanes makes `main` wait for them.  Inside a stream capture both become graph dependencies.
constexpr int kMaxLanes = 4;
int mtb_fork_lanes(cudaStream_t main, int lanes, cudaStream_t* out);
int mtb_join_lanes(cudaStream_t main, int lanes);

#define MTB_REQUIRE(cond, ...) \
  do { if (!(cond)) return mtb_fail(MTB_ERR_INVALID, __VA_ARGS__); } while (0)

#define MTB_CUDA(call) \
  do { cudaError_t e__ = (call); \
       if (e__ != cudaSuccess) return mtb_fail(MTB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__)); } while (0)

#define MTB_LAUNCH_CHECK(name) \
  do { cudaError_t e__ = cudaGetLastError(); \
       if (e__ != cudaSuccess) return mtb_fail(MTB_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); } while (0)

static inline int mtb_div_up(long long a, long long b) { return (int)((a + b - 1) / b); }

// Grid for a grid-stride bandwidth kernel: enough CTAs to fill the machine a few times over,
// as a multiple of the SM count, but never more than the work needs.
static inline int mtb_stream_grid(long long work_items, int threads, int ctas_per_sm = 8) {
  long long need = (work_items + threads - 1) / threads;
  long long cap = (long long)mtb_sm_count() * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

static inline bool mtb_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
