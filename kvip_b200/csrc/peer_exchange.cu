// Exchange of the per-rank TopK candidates of a sequence-sharded request over NVLink peer memory: one small kernel
// per rank writes its block into every rank's exchange block and raises a flag there; the merge kernel (topk.cu)
// waits for the flags. New on B200 (the reference has no multi-device code).
#include <cuda_runtime.h>
#include <cstring>
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kPeerThreads = 1024;
constexpr uint32_t kFlagsOffset = 256;   // bytes; the step counter sits at byte 0

__global__ void __launch_bounds__(kPeerThreads) peer_exchange(const KvipPeerExchangeArgs a) {
  __shared__ uint32_t step_now;
  uint8_t* own = reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(a.peer_block[a.rank]));
  if (threadIdx.x == 0) step_now = *reinterpret_cast<volatile uint32_t*>(own) + 1u;
  __syncthreads();
  const uint32_t step = step_now, half = step & 1u;
  const uint4* src = reinterpret_cast<const uint4*>(a.send);
  const uint32_t pieces = a.block_bytes >> 4;
  const uint64_t slot = KVIP_PEER_HEADER_BYTES + (static_cast<uint64_t>(half) * a.world + a.rank) * a.block_bytes;
  // every thread keeps its pieces in registers across the ranks: the send block is read once
  for (uint32_t p0 = threadIdx.x; p0 < pieces; p0 += kPeerThreads) {
    const uint4 v = src[p0];
    for (uint32_t r = 0; r < a.world; ++r)
      reinterpret_cast<uint4*>(static_cast<uintptr_t>(a.peer_block[r]) + slot)[p0] = v;
  }
  __threadfence_system();   // the candidates are visible on every GPU before any flag is
  __syncthreads();
  if (threadIdx.x < a.world) {
    volatile uint32_t* flag = reinterpret_cast<volatile uint32_t*>(static_cast<uintptr_t>(a.peer_block[threadIdx.x]) +
                                                                   kFlagsOffset) + a.rank;
    *flag = step;
  }
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(own) = step;
}

}  // namespace
}  // namespace kvip

extern "C" uint32_t kvip_b200_peer_exchange(const KvipPeerExchangeArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->send, "peer_exchange: null pointer");
  KVIP_REQUIRE(a->world >= 1 && a->world <= 8 && a->rank < a->world, "peer_exchange: 1..8 ranks");
  KVIP_REQUIRE(a->block_bytes && a->block_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(a->send) & 15) == 0,
               "peer_exchange: the candidate block must be 16-byte aligned and a multiple of 16 bytes");
  for (uint32_t r = 0; r < a->world; ++r)
    KVIP_REQUIRE(a->peer_block[r] && (a->peer_block[r] & 255) == 0, "peer_exchange: an exchange block is unmapped");
  kvip::peer_exchange<<<1, kvip::kPeerThreads, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("peer_exchange");
}

extern "C" uint32_t kvip_b200_peer_alloc(uint64_t bytes, void** block, uint8_t* handle) {
  KVIP_REQUIRE(block && handle && bytes >= KVIP_PEER_HEADER_BYTES, "peer_alloc: null pointer or a block without a header");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return kvip::check_launch("peer_alloc: cudaMalloc");
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    const uint32_t rc = kvip::check_launch("peer_alloc: IPC handle");
    cudaFree(p);
    return rc;
  }
  std::memcpy(handle, &h, sizeof(h));
  *block = p;
  return 0;
}

extern "C" uint32_t kvip_b200_peer_open(const uint8_t* handle, void** block) {
  KVIP_REQUIRE(handle && block, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  if (cudaIpcOpenMemHandle(block, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
    return kvip::check_launch("peer_open: cudaIpcOpenMemHandle");
  return 0;
}

extern "C" uint32_t kvip_b200_peer_close(void* block) {
  KVIP_REQUIRE(block, "peer_close: null pointer");
  if (cudaIpcCloseMemHandle(block) != cudaSuccess) return kvip::check_launch("peer_close: cudaIpcCloseMemHandle");
  return 0;
}

extern "C" uint32_t kvip_b200_peer_free(void* block) {
  KVIP_REQUIRE(block, "peer_free: null pointer");
  if (cudaFree(block) != cudaSuccess) return kvip::check_launch("peer_free: cudaFree");
  return 0;
}
