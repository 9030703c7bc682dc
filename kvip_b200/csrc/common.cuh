// Shared helpers for the kvip_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/kvip_b200.h"

namespace kvip {

constexpr uint32_t kTop = KVIP_TOPK;
constexpr uint32_t kSlots = KVIP_SLOTS;
constexpr uint32_t kLruSlots = KVIP_LRU_SLOTS;
constexpr uint32_t kChangeCapacity = KVIP_CHANGE_CAPACITY;
constexpr uint32_t kBlockTokens = KVIP_BLOCK_TOKENS;

// Host-side bookkeeping shared by the launchers (defined in api.cu).
void count_launch(uint32_t n = 1);
uint32_t check_launch(const char* what);
void set_error(const char* message);

// Per-device host bookkeeping. A function attribute (the dynamic shared-memory limit of a kernel) and the SM
// count belong to ONE device: a process that drives several GPUs configures every kernel once per device.
enum KernelSlot : uint32_t {
  kSlotLiFp8, kSlotLiBf16, kSlotTopkSelect, kSlotTopkMerge, kSlotTopkMergeCluster, kSlotTopkPivot, kSlotSplitEmit, kSlotSplitFallback,
  kSlotResolve, kSlotLidu, kSlotCount
};
// Raises the dynamic shared-memory limit of `kernel` on the current device the first time it is asked to there.
// Returns 0, or the launch-error code with the message set.
uint32_t raise_dynamic_smem(KernelSlot slot, const void* kernel, int bytes, const char* what);
uint32_t device_sm_count();   // SMs of the current device (148 when the query fails)

#define KVIP_REQUIRE(cond, msg)                 \
  do {                                          \
    if (!(cond)) {                              \
      ::kvip::set_error(msg);                   \
      return KVIP_BAD_ARGUMENT;                 \
    }                                           \
  } while (0)

// fp32 -> unsigned key with the same order (larger float = larger key).
// NaN sorts above +inf, like the reference's sortable-u16 map (score_common.h:66-97).
__host__ __device__ inline uint32_t sortable_key(float value) {
#ifdef __CUDA_ARCH__
  uint32_t bits = __float_as_uint(value);
#else
  union { float f; uint32_t u; } c; c.f = value; uint32_t bits = c.u;
#endif
  if ((bits & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// Round fp32 to bf16 with ties away from zero and widen back (CAST_ROUND,
// indexer_score.h:119-139; golden: workloads.py:233-235 "(bits + 0x8000) >> 16").
__host__ __device__ inline float bf16_away(float value) {
#ifdef __CUDA_ARCH__
  uint32_t bits = __float_as_uint(value);
  bits = (bits + 0x8000u) & 0xffff0000u;
  return __uint_as_float(bits);
#else
  union { float f; uint32_t u; } c; c.f = value;
  c.u = (c.u + 0x8000u) & 0xffff0000u;
  return c.f;
#endif
}

// Exclusive block-wide prefix sum for up to 1024 threads; `total` receives the sum.
// scratch: 33 words of shared memory. All threads of the block must call.
__device__ inline uint32_t block_exclusive_scan(uint32_t value, uint32_t* scratch, uint32_t* total) {
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  uint32_t scan = value;
#pragma unroll
  for (uint32_t d = 1; d < 32; d <<= 1) {
    uint32_t v = __shfl_up_sync(0xffffffffu, scan, d);
    if (lane >= d) scan += v;
  }
  __syncthreads();  // protects scratch reuse between consecutive calls
  if (lane == 31) scratch[warp] = scan;
  __syncthreads();
  if (warp == 0) {
    const uint32_t warps = (blockDim.x + 31u) >> 5;
    uint32_t v = lane < warps ? scratch[lane] : 0u;
#pragma unroll
    for (uint32_t d = 1; d < 32; d <<= 1) {
      uint32_t p = __shfl_up_sync(0xffffffffu, v, d);
      if (lane >= d) v += p;
    }
    scratch[lane] = v;
    if (lane == 31) scratch[32] = v;
  }
  __syncthreads();
  if (total) *total = scratch[32];
  return scan - value + (warp ? scratch[warp - 1] : 0u);
}

}  // namespace kvip
