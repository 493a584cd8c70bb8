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
//     event and is not handed out again until that event has completed.  pool_free(ptr)
//     (no stream) makes the block reusable at once, which is correct for this library's own
//     tensor_*_cuda ops because they all run on the legacy default stream: the next user's
//     kernels are ordered after the last user's.  Work on other streams must use
//     pool_free_async.
//   * debug mode (pool_set_debug(1), or LT_POOL_DEBUG=1 in the environment): every block
//     gets a 256-byte canary after the requested bytes, filled with 0xA5; pool_free checks
//     it and pool_check_canaries() checks every live block, reporting writes past the end
//     of an allocation on stderr.  This stands in for a memory sanitizer where none can run.
#include "luatorch_abi.h"

#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <unordered_map>
#include <vector>

namespace {

struct Block {
  void* ptr;
  size_t size;
  int device;
  cudaEvent_t ready;   // nullptr when reusable at once
  size_t user = 0;     // requested bytes (debug mode: the canary starts here)
};

constexpr size_t kCanaryBytes = 256;
constexpr unsigned char kCanaryByte = 0xA5;
int g_debug = -1;       // -1: read LT_POOL_DEBUG on first use
size_t g_overruns = 0;  // canaries found damaged so far

bool debug_on() {
  if (g_debug < 0) {
    const char* e = getenv("LT_POOL_DEBUG");
    g_debug = (e && e[0] == '1') ? 1 : 0;
  }
  return g_debug == 1;
}

// Returns true when the canary behind `b` is intact (device-to-host copy of 256 bytes).
bool canary_intact(const Block& b) {
  unsigned char host[kCanaryBytes];
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur != b.device) cudaSetDevice(b.device);
  const cudaError_t e = cudaMemcpy(host, static_cast<const char*>(b.ptr) + b.user, kCanaryBytes,
                                   cudaMemcpyDeviceToHost);
  if (cur != b.device) cudaSetDevice(cur);
  if (e != cudaSuccess) return false;
  for (size_t i = 0; i < kCanaryBytes; ++i)
    if (host[i] != kCanaryByte) return false;
  return true;
}

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
  std::lock_guard<std::mutex> lock(g_mu);
  const bool dbg = debug_on();
  const size_t size = round_up(bytes + (dbg ? kCanaryBytes : 0));
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  auto arm = [&](Block& b) {   // debug mode: lay the canary behind the user's bytes
    b.user = bytes;
    if (dbg) cudaMemset(static_cast<char*>(b.ptr) + bytes, kCanaryByte, kCanaryBytes);
  };
  DevicePool& p = g_pools[dev];
  for (auto it = p.free_blocks.lower_bound(size); it != p.free_blocks.end() && it->first <= 2 * size; ++it) {
    if (!block_ready(it->second)) continue;
    Block b = it->second;
    p.free_blocks.erase(it);
    g_cached -= b.size;
    arm(b);
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
  Block nb{ptr, size, dev, nullptr};
  arm(nb);
  g_live[ptr] = nb;
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
  if (debug_on() && !canary_intact(b)) {
    ++g_overruns;
    fprintf(stderr, "luatorch error: pool: write past the end of a %zu-byte block at %p (device %d)\n",
            b.user, b.ptr, b.device);
  }
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

// Extensions (debug mode, see the top of the file).
void pool_set_debug(int on) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_debug = on ? 1 : 0;
}
// Checks the canary of every live block; returns how many are damaged (0 when debug is off).
int pool_check_canaries(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!debug_on()) return 0;
  int bad = 0;
  for (auto& kv : g_live) {
    if (!canary_intact(kv.second)) {
      ++bad;
      fprintf(stderr, "luatorch error: pool: write past the end of a %zu-byte block at %p (device %d)\n",
              kv.second.user, kv.second.ptr, kv.second.device);
    }
  }
  return bad;
}
// Damaged canaries seen so far by pool_free / pool_free_async.
size_t pool_overruns_seen(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_overruns;
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
