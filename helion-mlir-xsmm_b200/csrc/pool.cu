// Device-side reuse pool: the B200 form of the reference's output pool
// (helion_mlir_backend/_compiler/output_pool.py). The reference keeps
// page-faulted host mappings so that a kernel's fresh output costs no faults;
// on the device the cost avoided is cudaMalloc/cudaFree, which synchronise the
// device. Policy kept from the reference (output_pool.py:60-69,142-202):
// reuse only for the same rounded size, whole 2 MiB units, at most max_bytes and
// 64 free blocks, oldest out first, a block larger than the limit is never kept,
// allocation failure frees every free block and retries once.
//
// Added for the device: stream-aware reuse. A freed block remembers the stream
// it was last used on and an event recorded there; a request on the same stream
// may take it at once (stream order protects it), a request on another stream
// only when the event has completed.
#include <atomic>
#include <list>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {
namespace {

constexpr size_t kGranule = size_t(2) << 20;
constexpr size_t kMaxFreeBlocks = 64;

struct Block {
  void* ptr = nullptr;
  size_t bytes = 0;
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t event = nullptr;
};

struct Pool {
  std::mutex mutex;
  std::list<Block> free_blocks;  // oldest first
  std::unordered_map<void*, Block> live;
  size_t free_bytes = 0;
  size_t live_bytes = 0;
  size_t max_bytes = size_t(2) << 30;
  uint64_t hits = 0, misses = 0;
};

Pool& pool() {
  static Pool* p = new Pool();  // never destroyed: frees may come at interpreter exit
  return *p;
}

void destroy(Block& b) {
  int current = -1;
  cudaGetDevice(&current);
  if (current != b.device) cudaSetDevice(b.device);
  if (b.event) cudaEventDestroy(b.event);
  cudaFree(b.ptr);
  if (current >= 0 && current != b.device) cudaSetDevice(current);
  cudaGetLastError();
}

// Caller holds the mutex.
void evict_over_limit(Pool& p) {
  while (!p.free_blocks.empty() && (p.free_bytes > p.max_bytes || p.free_blocks.size() > kMaxFreeBlocks)) {
    Block b = p.free_blocks.front();
    p.free_blocks.pop_front();
    p.free_bytes -= b.bytes;
    destroy(b);
  }
}

// Host-side failure injection for tests of the retry below: the next `count` device
// allocations of the pool fail with cudaErrorMemoryAllocation without reaching the
// driver (no device is driven out of memory to test this).
std::atomic<int> g_fail_allocations{0};

cudaError_t pool_malloc(void** ptr, size_t bytes) {
  int left = g_fail_allocations.load(std::memory_order_relaxed);
  while (left > 0) {
    if (g_fail_allocations.compare_exchange_weak(left, left - 1)) return cudaErrorMemoryAllocation;
  }
  return cudaMalloc(ptr, bytes);
}

void release_all(Pool& p) {
  for (Block& b : p.free_blocks) destroy(b);
  p.free_blocks.clear();
  p.free_bytes = 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_pool_alloc(size_t bytes, void* stream, void** out_ptr, int32_t* out_hit) {
  if (!out_ptr) return B200_E_NULL;
  *out_ptr = nullptr;
  if (out_hit) *out_hit = 0;
  if (bytes == 0) return B200_E_SHAPE;
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return -static_cast<int>(err);
  const size_t rounded = (bytes + kGranule - 1) / kGranule * kGranule;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Pool& p = pool();
  {
    std::lock_guard<std::mutex> lock(p.mutex);
    // Newest first: the block most likely still hot in L2 and on this stream.
    for (auto it = p.free_blocks.end(); it != p.free_blocks.begin();) {
      --it;
      if (it->bytes != rounded || it->device != device) continue;
      if (it->stream != s && it->event && cudaEventQuery(it->event) != cudaSuccess) {
        cudaGetLastError();
        continue;
      }
      Block b = *it;
      p.free_blocks.erase(it);
      p.free_bytes -= b.bytes;
      p.live[b.ptr] = b;
      p.live_bytes += b.bytes;
      ++p.hits;
      *out_ptr = b.ptr;
      if (out_hit) *out_hit = 1;
      return 0;
    }
    ++p.misses;
  }
  Block b;
  b.bytes = rounded;
  b.device = device;
  err = pool_malloc(&b.ptr, rounded);
  if (err != cudaSuccess) {
    cudaGetLastError();
    {
      std::lock_guard<std::mutex> lock(p.mutex);
      release_all(p);
    }
    err = pool_malloc(&b.ptr, rounded);
    if (err != cudaSuccess) {
      cudaGetLastError();
      return -static_cast<int>(err);
    }
  }
  {
    std::lock_guard<std::mutex> lock(p.mutex);
    p.live[b.ptr] = b;
    p.live_bytes += b.bytes;
  }
  *out_ptr = b.ptr;
  return 0;
}

extern "C" int b200_pool_free(void* ptr, void* stream) {
  if (!ptr) return 0;
  Pool& p = pool();
  Block b;
  {
    std::lock_guard<std::mutex> lock(p.mutex);
    auto it = p.live.find(ptr);
    if (it == p.live.end()) return B200_E_ARG;
    b = it->second;
    p.live.erase(it);
    p.live_bytes -= b.bytes;
  }
  int current = -1;
  cudaGetDevice(&current);
  if (current != b.device) cudaSetDevice(b.device);
  b.stream = static_cast<cudaStream_t>(stream);
  bool keep = b.bytes <= p.max_bytes;
  if (keep) {
    if (!b.event && cudaEventCreateWithFlags(&b.event, cudaEventDisableTiming) != cudaSuccess) {
      b.event = nullptr;
      keep = false;
    }
    if (keep && cudaEventRecord(b.event, b.stream) != cudaSuccess) keep = false;
  }
  cudaGetLastError();
  if (current >= 0 && current != b.device) cudaSetDevice(current);
  if (!keep) {
    destroy(b);
    return 0;
  }
  std::lock_guard<std::mutex> lock(p.mutex);
  p.free_blocks.push_back(b);
  p.free_bytes += b.bytes;
  evict_over_limit(p);
  return 0;
}

extern "C" int b200_pool_set_limit(size_t max_bytes) {
  Pool& p = pool();
  std::lock_guard<std::mutex> lock(p.mutex);
  p.max_bytes = max_bytes;
  evict_over_limit(p);
  return 0;
}

extern "C" int b200_pool_release(void) {
  Pool& p = pool();
  std::lock_guard<std::mutex> lock(p.mutex);
  release_all(p);
  return 0;
}

extern "C" int b200_pool_stats(b200_pool_stats_t* out) {
  if (!out) return B200_E_NULL;
  Pool& p = pool();
  std::lock_guard<std::mutex> lock(p.mutex);
  out->hits = p.hits;
  out->misses = p.misses;
  out->free_blocks = p.free_blocks.size();
  out->free_bytes = p.free_bytes;
  out->max_bytes = p.max_bytes;
  out->live_blocks = p.live.size();
  out->live_bytes = p.live_bytes;
  return 0;
}

extern "C" int b200_pool_inject_alloc_failures(int32_t count) {
  if (count < 0) return B200_E_ARG;
  g_fail_allocations.store(count, std::memory_order_relaxed);
  return 0;
}
