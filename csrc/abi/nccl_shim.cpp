// luatorch_nccl_* entry points (lua/luatorch/distributed/init.lua:17-21) WITHOUT NCCL: the
// single-process, one-pointer-per-device calling convention of the reference wrapper
// (csrc/distributed/nccl_wrapper.cu:37-135) is served by this repository's own peer-memory
// kernels (csrc/comm/comm_kernels.cu).  Every device enables peer access to the others; a
// call launches one kernel per device, all of them working on the same table of peer
// addresses, and returns after every device's stream has drained (the reference also blocks
// the host after each collective).  Devices without peer access fall back to a host-staged
// reduction.  Return codes as in the reference: 0 ok, -1 error.
#include "luatorch_abi.h"

#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>
#include <vector>

#include "../comm/comm_kernels.h"

namespace {

constexpr int kMax = 16;
struct DevState {
  cudaStream_t stream = nullptr;
  uint32_t* pad = nullptr;        // signal pad (256 uint32)
  int* status = nullptr;          // 8 ints
  uint64_t* ptr_table = nullptr;  // device copy of the pointer table
  uint64_t* pad_table = nullptr;  // device copy of the signal-pad table
};
DevState g_dev[kMax];
int g_n = 0;
bool g_peer_ok = false;
uint32_t g_epoch = 0;

int fail(const char* what, cudaError_t e) {
  fprintf(stderr, "luatorch nccl error: %s: %s\n", what, cudaGetErrorString(e));
  return -1;
}

int host_staged_allreduce(float** ptrs, int64_t count, int n) {
  std::vector<float> acc((size_t)count, 0.0f), tmp((size_t)count);
  for (int d = 0; d < n; ++d) {
    cudaSetDevice(d);
    if (cudaMemcpy(tmp.data(), ptrs[d], (size_t)count * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    for (int64_t i = 0; i < count; ++i) acc[(size_t)i] += tmp[(size_t)i];
  }
  for (int64_t i = 0; i < count; ++i) acc[(size_t)i] /= (float)n;
  for (int d = 0; d < n; ++d) {
    cudaSetDevice(d);
    if (cudaMemcpy(ptrs[d], acc.data(), (size_t)count * 4, cudaMemcpyHostToDevice) != cudaSuccess) return -1;
  }
  return 0;
}

int check_status(int n) {
  int bad = 0;
  for (int d = 0; d < n; ++d) {
    int st[8] = {0};
    cudaSetDevice(d);
    cudaMemcpy(st, g_dev[d].status, sizeof(st), cudaMemcpyDeviceToHost);
    if (st[0] != 0) {
      fprintf(stderr, "luatorch nccl error: device %d: wait expired (code %d, epoch %d, phase %d, peer %d)\n", d,
              st[0], st[2], st[3], st[4]);
      cudaMemset(g_dev[d].status, 0, sizeof(st));
      bad = 1;
    }
  }
  return bad ? -1 : 0;
}

}  // namespace

extern "C" {

int luatorch_nccl_get_gpu_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

int luatorch_nccl_init(int num_gpus) {
  if (g_n) return 0;
  int avail = luatorch_nccl_get_gpu_count();
  if (num_gpus < 1 || num_gpus > avail || num_gpus > kMax) {
    fprintf(stderr, "luatorch nccl error: requested %d gpus, %d available\n", num_gpus, avail);
    return -1;
  }
  g_peer_ok = true;
  for (int d = 0; d < num_gpus; ++d) {
    cudaSetDevice(d);
    for (int p = 0; p < num_gpus; ++p) {
      if (p == d) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, d, p);
      if (!can) { g_peer_ok = false; continue; }
      cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) g_peer_ok = false;
      (void)cudaGetLastError();
    }
    DevState& s = g_dev[d];
    // A blocking stream: it is ordered after work already queued on the device's legacy default
    // stream, where every tensor_*_cuda op of this library runs, so a collective never reads a
    // buffer whose producing kernel is still running (the reference creates its streams the
    // same way, csrc/distributed/nccl_wrapper.cu:62-65).
    cudaError_t e = cudaStreamCreate(&s.stream);
    if (e != cudaSuccess) return fail("stream create", e);
    if (cudaMalloc(&s.pad, 1024) != cudaSuccess || cudaMalloc(&s.status, 64) != cudaSuccess ||
        cudaMalloc(&s.ptr_table, kMax * 8) != cudaSuccess || cudaMalloc(&s.pad_table, kMax * 8) != cudaSuccess)
      return fail("device allocation", cudaGetLastError());
    cudaMemset(s.pad, 0, 1024);
    cudaMemset(s.status, 0, 64);
  }
  uint64_t pads[kMax];
  for (int d = 0; d < num_gpus; ++d) pads[d] = (uint64_t)(uintptr_t)g_dev[d].pad;
  for (int d = 0; d < num_gpus; ++d) {
    cudaSetDevice(d);
    cudaMemcpy(g_dev[d].pad_table, pads, sizeof(uint64_t) * num_gpus, cudaMemcpyHostToDevice);
    cudaDeviceSynchronize();
  }
  g_n = num_gpus;
  cudaSetDevice(0);
  return 0;
}

int luatorch_nccl_allreduce(float** ptrs, int64_t count, int num_gpus) {
  if (!g_n || num_gpus != g_n || !ptrs || count <= 0) {
    fprintf(stderr, "luatorch nccl error: allreduce before init or with a different gpu count\n");
    return -1;
  }
  if (num_gpus == 1) return 0;
  bool same = true;                       // the reference's DDP passes one pointer n times
  for (int d = 1; d < num_gpus; ++d) same = same && ptrs[d] == ptrs[0];
  if (same) return 0;                     // the average of n copies of x is x
  if (!g_peer_ok) return host_staged_allreduce(ptrs, count, num_gpus);
  // the peer kernel moves 16-byte vectors: a float* that is not 16-byte aligned takes the
  // host-staged path instead of raising a misaligned-address error on the device
  for (int d = 0; d < num_gpus; ++d)
    if ((uintptr_t)ptrs[d] & 15) return host_staged_allreduce(ptrs, count, num_gpus);
  const int64_t gran = 4 * (int64_t)num_gpus;
  const int64_t main = count / gran * gran;
  uint64_t table[kMax];
  for (int d = 0; d < num_gpus; ++d) table[d] = (uint64_t)(uintptr_t)ptrs[d];
  if (main > 0) {
    const uint32_t epoch = ++g_epoch;
    for (int d = 0; d < num_gpus; ++d) {
      cudaSetDevice(d);
      DevState& s = g_dev[d];
      cudaMemcpyAsync(s.ptr_table, table, sizeof(uint64_t) * num_gpus, cudaMemcpyHostToDevice, s.stream);
      cudaError_t e = lt::peer_allreduce(s.ptr_table, s.pad_table, d, num_gpus, 0, main, lt::DT_F32,
                                         1.0f / (float)num_gpus, epoch, s.status, s.stream);
      if (e != cudaSuccess) return fail("allreduce launch", e);
    }
  }
  for (int d = 0; d < num_gpus; ++d) {
    cudaSetDevice(d);
    cudaStreamSynchronize(g_dev[d].stream);
  }
  int rc = main > 0 ? check_status(num_gpus) : 0;
  if (rc == 0 && main < count) {          // fewer than 4*n trailing elements: host staged
    float* tails[kMax];
    for (int d = 0; d < num_gpus; ++d) tails[d] = ptrs[d] + main;
    rc = host_staged_allreduce(tails, count - main, num_gpus);
  }
  cudaSetDevice(0);
  return rc;
}

int luatorch_nccl_broadcast(float** ptrs, int64_t count, int root, int num_gpus) {
  if (!g_n || num_gpus != g_n || !ptrs || count <= 0 || root < 0 || root >= num_gpus) {
    fprintf(stderr, "luatorch nccl error: bad broadcast arguments\n");
    return -1;
  }
  if (num_gpus == 1) return 0;
  if (!g_peer_ok) {
    std::vector<float> tmp((size_t)count);
    cudaSetDevice(root);
    if (cudaMemcpy(tmp.data(), ptrs[root], (size_t)count * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    for (int d = 0; d < num_gpus; ++d) {
      if (d == root) continue;
      cudaSetDevice(d);
      if (cudaMemcpy(ptrs[d], tmp.data(), (size_t)count * 4, cudaMemcpyHostToDevice) != cudaSuccess) return -1;
    }
    cudaSetDevice(0);
    return 0;
  }
  uint64_t table[kMax];
  for (int d = 0; d < num_gpus; ++d) table[d] = (uint64_t)(uintptr_t)ptrs[d];
  const uint32_t epoch = ++g_epoch;
  for (int d = 0; d < num_gpus; ++d) {
    cudaSetDevice(d);
    DevState& s = g_dev[d];
    cudaMemcpyAsync(s.ptr_table, table, sizeof(uint64_t) * num_gpus, cudaMemcpyHostToDevice, s.stream);
    cudaError_t e = lt::peer_broadcast(s.ptr_table, s.pad_table, d, num_gpus, root, 0, count * 4, epoch, s.status,
                                       s.stream);
    if (e != cudaSuccess) return fail("broadcast launch", e);
  }
  for (int d = 0; d < num_gpus; ++d) {
    cudaSetDevice(d);
    cudaStreamSynchronize(g_dev[d].stream);
  }
  const int rc = check_status(num_gpus);
  cudaSetDevice(0);
  return rc;
}

void luatorch_nccl_destroy(void) {
  for (int d = 0; d < g_n; ++d) {
    cudaSetDevice(d);
    DevState& s = g_dev[d];
    if (s.stream) cudaStreamDestroy(s.stream);
    cudaFree(s.pad); cudaFree(s.status); cudaFree(s.ptr_table); cudaFree(s.pad_table);
    s = DevState();
  }
  g_n = 0;
  g_epoch = 0;
  cudaSetDevice(0);
}

}  // extern "C"
