// The runtime half of the boundary: device memory pool, host<->device copies, streams, events and
// whole-step CUDA graphs, behind the same C ABI as the kernels.  It plays the role of the reference's
// mytorch/backends/cuda/memory_allocator.py:16-51 (a caching allocator keyed by size) and of the stream /
// memcpy plumbing in mytorch/backends/cuda/env.py:61-94 and :524-580.
//
// Pool.  Freed blocks are kept per device in size-keyed free lists and handed out again to requests of
// (nearly) the same size, so a training step that repeats the same allocation pattern reuses the same
// addresses step after step and never reaches cudaMalloc after the first step.  Nothing is split or
// merged.  The pool does no stream tracking: a block returns to its free list the moment it is freed,
// which is safe for memory that is only touched by work on the device's one compute stream (work is
// stream ordered).  Memory handed to another stream must be kept alive by its owner until that stream is done.
//
// Graphs.  Between mtb_graph_begin_capture and mtb_graph_end_capture every block handed out is tagged
// with the graph being captured.  Such a block may be reused inside the same capture (its earlier use is
// ordered before the later one on the captured stream) but never returns to the general pool while the
// graph exists, because every replay writes it again.  mtb_graph_destroy releases the graph's blocks.
#include "common.cuh"
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Block {
  size_t size;
  int device;
  unsigned long long graph;  // 0: ordinary block; otherwise the capture that handed it out
};

struct DevicePool {
  std::multimap<size_t, void*> free_blocks;                                  // general pool
  std::unordered_map<unsigned long long, std::multimap<size_t, void*>> graph_free;  // freed while their graph exists
  size_t reserved = 0, in_use = 0;
};

struct Runtime {
  std::mutex mu;
  std::unordered_map<void*, Block> blocks;  // every block the pool owns, free or not
  std::map<int, DevicePool> pools;
  unsigned long long capturing = 0;         // graph id of the capture in progress (one at a time)
  unsigned long long next_graph = 1;
  std::unordered_map<void*, unsigned long long> graph_of_exec;
};

Runtime& rt() {
  static Runtime* r = new Runtime();  // never destroyed: frees may arrive during interpreter shutdown
  return *r;
}

size_t round_size(size_t n) {
  if (n == 0) n = 1;
  const size_t g = n <= (1u << 20) ? 512 : (n <= (64u << 20) ? (size_t)1 << 16 : (size_t)1 << 21);
  return (n + g - 1) / g * g;
}

// A free block is good for a request if it wastes at most 1/8 of itself (or 64 KiB).
void* take_fit(std::multimap<size_t, void*>& list, size_t want, size_t* got) {
  auto it = list.lower_bound(want);
  if (it == list.end()) return nullptr;
  const size_t slack = it->first - want;
  if (slack > it->first / 8 && slack > (1u << 16)) return nullptr;
  void* p = it->second;
  *got = it->first;
  list.erase(it);
  return p;
}

int trim_locked(DevicePool& pool) {
  for (auto& kv : pool.free_blocks) {
    cudaFree(kv.second);
    pool.reserved -= kv.first;
    rt().blocks.erase(kv.second);
  }
  pool.free_blocks.clear();
  return MTB_OK;
}

}  // namespace

// Device memory from the pool of the current device (NULL on failure, see mtb_last_error).
MTB_API void* mtb_malloc(long long nbytes) {
  if (nbytes < 0) { mtb_fail(MTB_ERR_INVALID, "mtb_malloc: negative size"); return nullptr; }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { mtb_fail(MTB_ERR_CUDA, "mtb_malloc: no current device"); return nullptr; }
  const size_t want = round_size((size_t)nbytes);
  Runtime& r = rt();
  std::lock_guard<std::mutex> lock(r.mu);
  DevicePool& pool = r.pools[dev];
  size_t got = 0;
  void* p = nullptr;
  if (r.capturing) p = take_fit(pool.graph_free[r.capturing], want, &got);
  if (!p) p = take_fit(pool.free_blocks, want, &got);
  if (!p) {
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {  // give back what is cached and try once more
      cudaGetLastError();
      trim_locked(pool);
      e = cudaMalloc(&p, want);
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      mtb_fail(MTB_ERR_CUDA, "mtb_malloc: cudaMalloc of %zu bytes failed: %s", want, cudaGetErrorString(e));
      return nullptr;
    }
    got = want;
    pool.reserved += want;
    r.blocks[p] = Block{want, dev, 0};
  }
  r.blocks[p].graph = r.capturing;
  pool.in_use += got;
  return p;
}

MTB_API int mtb_free(void* ptr) {
  if (!ptr) return MTB_OK;
  Runtime& r = rt();
  std::lock_guard<std::mutex> lock(r.mu);
  auto it = r.blocks.find(ptr);
  if (it == r.blocks.end()) return mtb_fail(MTB_ERR_INVALID, "mtb_free: %p was not allocated by mtb_malloc", ptr);
  Block& b = it->second;
  DevicePool& pool = r.pools[b.device];
  pool.in_use -= b.size;
  if (b.graph) pool.graph_free[b.graph].emplace(b.size, ptr);
  else pool.free_blocks.emplace(b.size, ptr);
  return MTB_OK;
}

// Bytes the pool holds from the driver / bytes currently handed out, on the current device.
MTB_API long long mtb_pool_reserved_bytes() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(rt().mu);
  return (long long)rt().pools[dev].reserved;
}
MTB_API long long mtb_pool_in_use_bytes() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(rt().mu);
  return (long long)rt().pools[dev].in_use;
}
// Return every cached free block of the current device to the driver (synchronises the device).
MTB_API int mtb_pool_trim() {
  int dev = 0;
  MTB_CUDA(cudaGetDevice(&dev));
  MTB_CUDA(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(rt().mu);
  return trim_locked(rt().pools[dev]);
}

MTB_API int mtb_set_device(int device) { MTB_CUDA(cudaSetDevice(device)); return MTB_OK; }
MTB_API int mtb_get_device(int* device) { MTB_CUDA(cudaGetDevice(device)); return MTB_OK; }
MTB_API int mtb_device_count(int* count) { MTB_CUDA(cudaGetDeviceCount(count)); return MTB_OK; }
MTB_API int mtb_device_synchronize() { MTB_CUDA(cudaDeviceSynchronize()); return MTB_OK; }
MTB_API int mtb_mem_get_info(long long* free_bytes, long long* total_bytes) {
  size_t f = 0, t = 0;
  MTB_CUDA(cudaMemGetInfo(&f, &t));
  if (free_bytes) *free_bytes = (long long)f;
  if (total_bytes) *total_bytes = (long long)t;
  return MTB_OK;
}

// ---- copies (asynchronous on `stream`; host memory should be pinned for a truly asynchronous copy) ----
MTB_API int mtb_memcpy_h2d_async(void* dst, const void* src_host, long long nbytes, void* stream) {
  MTB_REQUIRE(nbytes >= 0 && ((dst && src_host) || nbytes == 0), "memcpy_h2d: bad arguments");
  if (nbytes) MTB_CUDA(cudaMemcpyAsync(dst, src_host, (size_t)nbytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return MTB_OK;
}
MTB_API int mtb_memcpy_d2h_async(void* dst_host, const void* src, long long nbytes, void* stream) {
  MTB_REQUIRE(nbytes >= 0 && ((dst_host && src) || nbytes == 0), "memcpy_d2h: bad arguments");
  if (nbytes) MTB_CUDA(cudaMemcpyAsync(dst_host, src, (size_t)nbytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return MTB_OK;
}
MTB_API int mtb_memcpy_d2d_async(void* dst, const void* src, long long nbytes, void* stream) {
  MTB_REQUIRE(nbytes >= 0 && ((dst && src) || nbytes == 0), "memcpy_d2d: bad arguments");
  if (nbytes) MTB_CUDA(cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDefault, (cudaStream_t)stream));
  return MTB_OK;
}
MTB_API int mtb_memset_async(void* dst, int value, long long nbytes, void* stream) {
  MTB_REQUIRE(nbytes >= 0 && (dst || nbytes == 0), "memset: bad arguments");
  if (nbytes) MTB_CUDA(cudaMemsetAsync(dst, value, (size_t)nbytes, (cudaStream_t)stream));
  return MTB_OK;
}
MTB_API void* mtb_host_alloc_pinned(long long nbytes) {
  void* p = nullptr;
  cudaError_t e = cudaHostAlloc(&p, (size_t)(nbytes > 0 ? nbytes : 1), cudaHostAllocDefault);
  if (e != cudaSuccess) { mtb_fail(MTB_ERR_CUDA, "host_alloc_pinned: %s", cudaGetErrorString(e)); return nullptr; }
  return p;
}
MTB_API int mtb_host_free_pinned(void* p) {
  if (p) MTB_CUDA(cudaFreeHost(p));
  return MTB_OK;
}

// ---- streams and events ----
MTB_API void* mtb_stream_create() {
  cudaStream_t s = nullptr;
  cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (e != cudaSuccess) { mtb_fail(MTB_ERR_CUDA, "stream_create: %s", cudaGetErrorString(e)); return nullptr; }
  return s;
}
MTB_API int mtb_stream_destroy(void* s) { if (s) MTB_CUDA(cudaStreamDestroy((cudaStream_t)s)); return MTB_OK; }
MTB_API int mtb_stream_synchronize(void* s) { MTB_CUDA(cudaStreamSynchronize((cudaStream_t)s)); return MTB_OK; }
MTB_API int mtb_stream_wait_event(void* s, void* ev) { MTB_CUDA(cudaStreamWaitEvent((cudaStream_t)s, (cudaEvent_t)ev, 0)); return MTB_OK; }
MTB_API void* mtb_event_create(int timing) {
  cudaEvent_t ev = nullptr;
  cudaError_t e = cudaEventCreateWithFlags(&ev, timing ? cudaEventDefault : cudaEventDisableTiming);
  if (e != cudaSuccess) { mtb_fail(MTB_ERR_CUDA, "event_create: %s", cudaGetErrorString(e)); return nullptr; }
  return ev;
}
MTB_API int mtb_event_destroy(void* ev) { if (ev) MTB_CUDA(cudaEventDestroy((cudaEvent_t)ev)); return MTB_OK; }
MTB_API int mtb_event_record(void* ev, void* s) { MTB_CUDA(cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)s)); return MTB_OK; }
MTB_API int mtb_event_synchronize(void* ev) { MTB_CUDA(cudaEventSynchronize((cudaEvent_t)ev)); return MTB_OK; }
MTB_API int mtb_event_elapsed_ms(void* start, void* end, float* ms) {
  MTB_REQUIRE(ms, "event_elapsed_ms: no output");
  MTB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end));
  return MTB_OK;
}

// ---- whole-step graphs ----
// Start recording everything enqueued on `stream` (and on streams that fork from it through events) into
// a graph instead of running it.  Relaxed capture mode: other host threads (a collective library's
// watchdog, say) may keep making CUDA calls, and the pool may still reach cudaMalloc for a size it has not seen.
MTB_API int mtb_graph_begin_capture(void* stream) {
  Runtime& r = rt();
  {
    std::lock_guard<std::mutex> lock(r.mu);
    if (r.capturing) return mtb_fail(MTB_ERR_INVALID, "graph_begin_capture: a capture is already in progress");
    r.capturing = r.next_graph++;
  }
  cudaError_t e = cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeRelaxed);
  if (e != cudaSuccess) {
    std::lock_guard<std::mutex> lock(r.mu);
    r.capturing = 0;
    return mtb_fail(MTB_ERR_CUDA, "cudaStreamBeginCapture: %s", cudaGetErrorString(e));
  }
  return MTB_OK;
}

MTB_API int mtb_graph_end_capture(void* stream, void** graph_exec_out) {
  MTB_REQUIRE(graph_exec_out, "graph_end_capture: no output");
  Runtime& r = rt();
  unsigned long long id;
  {
    std::lock_guard<std::mutex> lock(r.mu);
    id = r.capturing;
    r.capturing = 0;
  }
  MTB_REQUIRE(id != 0, "graph_end_capture: no capture in progress");
  cudaGraph_t graph = nullptr;
  MTB_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return mtb_fail(MTB_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  {
    std::lock_guard<std::mutex> lock(r.mu);
    r.graph_of_exec[exec] = id;
  }
  *graph_exec_out = exec;
  return MTB_OK;
}

MTB_API int mtb_graph_launch(void* graph_exec, void* stream) {
  MTB_REQUIRE(graph_exec, "graph_launch: no graph");
  MTB_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
  return MTB_OK;
}

// Destroys the executable graph (the caller has made sure no replay is in flight) and hands the blocks
// that only the graph kept alive back to the pool.
MTB_API int mtb_graph_destroy(void* graph_exec) {
  if (!graph_exec) return MTB_OK;
  Runtime& r = rt();
  unsigned long long id = 0;
  {
    std::lock_guard<std::mutex> lock(r.mu);
    auto it = r.graph_of_exec.find(graph_exec);
    if (it == r.graph_of_exec.end()) return mtb_fail(MTB_ERR_INVALID, "graph_destroy: unknown graph");
    id = it->second;
    r.graph_of_exec.erase(it);
    for (auto& kv : r.blocks)
      if (kv.second.graph == id) kv.second.graph = 0;  // blocks still in use return to the general pool when freed
    for (auto& dp : r.pools) {
      auto gf = dp.second.graph_free.find(id);
      if (gf == dp.second.graph_free.end()) continue;
      for (auto& b : gf->second) dp.second.free_blocks.emplace(b.first, b.second);
      dp.second.graph_free.erase(gf);
    }
  }
  MTB_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
  return MTB_OK;
}
