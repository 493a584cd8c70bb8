// Hand-written collectives over NVLink / NVSwitch peer memory, fused with the optimizer.
//
// They replace the reference's NCCL wrapper (csrc/distributed/nccl_wrapper.cu:88-135: one
// blocking ncclAllReduce per parameter tensor followed by a host stream synchronise, and an
// ncclBroadcast) and the separate per-tensor Adam launches that follow it
// (lua/luatorch/distributed/ddp.lua:48-61, lua/luatorch/optim/adamw.lua:51-102).
//
// Every rank passes the same tables of peer-mapped addresses (one entry per rank, entry
// `rank` being its own local buffer) and a signal pad per rank: uint32 slots
// [0, 16) "start" and [16, 32) "done", written by peers with release.sys stores and read with
// acquire.sys loads, word 32 a block ticket, word 33 the pad's own collective counter.
// `epoch` increases by one per collective on every rank; a caller that passes 0 lets the
// kernels count for themselves in word 33 (all collectives on one pad must then do so, and
// must be ordered on one stream), which is what makes a captured CUDA graph replayable.
// Every wait is bounded; on expiry the kernel records
// {code, rank, epoch, phase, peer, seen} in `status` (8 ints) and returns without touching
// data it could not prove complete.  Data moves with plain vector ld/st only.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../kernels/ops.h"

namespace lt {

enum CommMode : int {
  // Every rank sums all peers' gradients for the whole range and applies AdamW to its full
  // replica in registers (one launch; best for small buckets).
  COMM_ONE_SHOT_REPLICATED = 0,
  // Rank r reduces slice r, applies AdamW to slice r of master / m / v (sharded optimizer
  // state) and stores the updated bf16 parameters of the slice into every peer's shadow
  // arena (reduce-scatter + shard AdamW + parameter all-gather by push, one launch).
  COMM_TWO_SHOT_SHARDED = 1,
};

enum CommOpt : int {
  COMM_OPT_ADAMW = 0,   // AdamW / Adam on master, m, v
  COMM_OPT_SGD = 1,     // SGD with momentum: `m` is the velocity (may be null: plain SGD), `v` unused
};

struct CommAdamArgs {
  const uint64_t* grad_ptrs = nullptr;    // [world] device table: bf16 gradient arenas
  const uint64_t* signal_ptrs = nullptr;  // [world] device table: signal pads
  const uint64_t* shadow_ptrs = nullptr;  // [world] device table: bf16 shadow-parameter arenas
  int rank = 0, world = 1;
  int64_t elem_offset = 0;                // first arena element of the bucket
  int64_t n = 0;                          // elements in the bucket (multiple of 8 * world)
  // NVLS (sharded mode only): multicast addresses of the gradient and shadow arenas.  With
  // grad_mc the slice is read with multimem.ld_reduce, with shadow_mc the update is published
  // with multimem.st; null = plain peer loads / stores.
  const void* grad_mc = nullptr;
  void* shadow_mc = nullptr;
  float* master = nullptr;                // local fp32 optimizer state
  float* m = nullptr;
  float* v = nullptr;
  // Index into master / m / v of the first element this rank updates.  -1: the state arrays
  // are full length and indexed like the gradients; >= 0: they hold only this rank's shards
  // (memory-sharded optimizer state) and this bucket's shard starts there.
  int64_t state_base = -1;
  int opt_kind = COMM_OPT_ADAMW;
  float momentum = 0.0f;                  // COMM_OPT_SGD
  int nesterov = 0;
  const int64_t* seg_end = nullptr;       // weight-decay segments in arena coordinates
  const float* seg_wd = nullptr;
  int nseg = 0;
  AdamArgs adam{};                        // grad_scale carries 1/world (and 1/loss-scale)
  uint32_t epoch = 0;                     // 0: the kernel numbers itself from its signal pad
  int mode = COMM_ONE_SHOT_REPLICATED;
  int max_blocks = 0;                     // 0 = default
  int* status = nullptr;                  // [8] device ints, zero when healthy
};

cudaError_t allreduce_adamw(const CommAdamArgs& a, cudaStream_t stream);

// root's bytes [byte_offset, byte_offset + nbytes) of its buffer -> same range of every rank.
cudaError_t peer_broadcast(const uint64_t* buf_ptrs, const uint64_t* signal_ptrs, int rank,
                           int world, int root, int64_t byte_offset, int64_t nbytes,
                           uint32_t epoch, int* status, cudaStream_t stream);

// In-place sum (times `scale`) of elements [elem_offset, elem_offset + n) across ranks.
// dtype: DT_F32 or DT_BF16 (fp32 accumulation).  n must be a multiple of 8 * world.
cudaError_t peer_allreduce(const uint64_t* buf_ptrs, const uint64_t* signal_ptrs, int rank,
                           int world, int64_t elem_offset, int64_t n, int dtype, float scale,
                           uint32_t epoch, int* status, cudaStream_t stream);

// Waits (bounded by `budget_cycles`) until *flag >= expected; on expiry writes code 100 into
// status[0] and returns.  Used by the failure-detection tests: a flag nobody sets makes the
// wait run out and the context stays usable.
cudaError_t wait_flag_bounded(const uint32_t* flag, uint32_t expected, int64_t budget_cycles,
                              int* status, cudaStream_t stream);

uint64_t comm_launch_count();

}  // namespace lt
