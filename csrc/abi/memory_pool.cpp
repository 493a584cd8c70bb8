// Caching device-memory pool behind the pool_* ABI (counterpart of the reference's
// csrc/cuda/memory_pool.cu).
//
// What it keeps from the reference: the ABI, 512-byte minimum / power-of-two size classes for
// small requests, "clear the cache and retry once" on allocation failure, cudaFree for
// pointers it does not know, and the two byte counters.
// What it does differently, for multi-GPU and async use on a 180 GB part:
//   * one set of free lists PER DEVICE (the reference keeps a single list for all GPUs, so a
//     block cached on one device can be handed out on another);
//   * O(1) bins instead of a linear scan of a linked list: 512 B .. 1 MiB in powers of two,
//     larger requests rounded to 2 MiB and served best-fit from an ordered map (a block at
//     most 2x the request is accepted, as in the reference);
//   * stream-ordered reuse: a block released with pool_free_async(ptr, stream) carries an
//     event and is not handed out again until that event has completed.
#include "luatorch_abi.h"

#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <stdio.h>
#include <unordered_map>
#include <vector>

namespace {

struct Block {
  void* ptr;
  size_t size;
  int device;
  cudaEvent_t ready;   // nullptr when reusable at once
};

constexpr size_t kMinBlock = 512;
constexpr size_t kSmallMax = 1 << 20;
constexpr size_t kLargeRound = 2 << 20;
constexpr int kMaxDevices = 64;

struct DevicePool {
  std::multimap<size_t, Block> free_blocks;   // size -> block
};

std::mutex g_mu;
DevicePool g_pools[kMaxDevices];
std::unordered_map<void*, Block> g_live;      // blocks handed out
size_t g_allocated = 0;                       // bytes obtained from cudaMalloc and still owned
size_t g_cached = 0;                          // bytes sitting in free lists
bool g_init = false;

size_t round_up(size_t bytes) {
  if (bytes < kMinBlock) return kMinBlock;
  if (bytes <= kSmallMax) {
    size_t s = kMinBlock;
    while (s < bytes) s <<= 1;
    return s;
  }
  return (bytes + kLargeRound - 1) / kLargeRound * kLargeRound;
}

bool block_ready(Block& b) {
  if (!b.ready) return true;
  if (cudaEventQuery(b.ready) == cudaSuccess) {
    cudaEventDestroy(b.ready);
    b.ready = nullptr;
    return true;
  }
  (void)cudaGetLastError();   // cudaErrorNotReady is not an error here
  return false;
}

void release_cached_locked(int device) {
  DevicePool& p = g_pools[device];
  for (auto& kv : p.free_blocks) {
    Block& b = kv.second;
    if (b.ready) { cudaEventSynchronize(b.ready); cudaEventDestroy(b.ready); }
    cudaFree(b.ptr);
    g_allocated -= b.size;
    g_cached -= b.size;
  }
  p.free_blocks.clear();
}

}  // namespace

extern "C" {

void pool_init(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_init = true;
}

void* pool_alloc(size_t bytes) {
  const size_t size = round_up(bytes);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  DevicePool& p = g_pools[dev];
  for (auto it = p.free_blocks.lower_bound(size); it != p.free_blocks.end() && it->first <= 2 * size; ++it) {
    if (!block_ready(it->second)) continue;
    Block b = it->second;
    p.free_blocks.erase(it);
    g_cached -= b.size;
    g_live[b.ptr] = b;
    return b.ptr;
  }
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, size);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    release_cached_locked(dev);          // give the cache back to the driver and retry once
    e = cudaMalloc(&ptr, size);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      fprintf(stderr, "luatorch error: pool_alloc failed for %zu bytes: %s\n", size, cudaGetErrorString(e));
      return nullptr;
    }
  }
  g_allocated += size;
  g_live[ptr] = Block{ptr, size, dev, nullptr};
  return ptr;
}

// Extension: release a block whose last use was enqueued on `stream`.
void pool_free_async(void* ptr, void* stream) {
  if (!ptr) return;
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_live.find(ptr);
  if (it == g_live.end()) {
    cudaFree(ptr);                        // not ours: hand it to the driver, as the reference does
    return;
  }
  Block b = it->second;
  g_live.erase(it);
  if (stream != nullptr) {
    int cur = 0;
    cudaGetDevice(&cur);
    if (cur != b.device) cudaSetDevice(b.device);
    if (cudaEventCreateWithFlags(&b.ready, cudaEventDisableTiming) == cudaSuccess)
      cudaEventRecord(b.ready, (cudaStream_t)stream);
    else
      b.ready = nullptr;
    if (cur != b.device) cudaSetDevice(cur);
  }
  g_pools[b.device].free_blocks.emplace(b.size, b);
  g_cached += b.size;
}

void pool_free(void* ptr) { pool_free_async(ptr, nullptr); }

void pool_clear(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  for (int d = 0; d < kMaxDevices; ++d) {
    if (g_pools[d].free_blocks.empty()) continue;
    cudaSetDevice(d);
    release_cached_locked(d);
  }
  cudaSetDevice(cur);
}

size_t pool_allocated_bytes(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_allocated;
}
size_t pool_cached_bytes(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_cached;
}
size_t cuda_memory_allocated(void) { return pool_allocated_bytes(); }
size_t cuda_memory_cached(void) { return pool_cached_bytes(); }

}  // extern "C"
