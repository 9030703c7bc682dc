// Index exchange: keep "physical Index position p < resident describes hot slot p" after a
// round of slot assignments. One CTA of 1024 threads per request.
//
// Same plan as ApplyBatch / ApplyDenseBatch (op_kernel/shadow_exchange_parallel.h:27-198),
// driven per query like Consumer (streaming.cpp:205-274): events (orig position, dst slot) in
// rank order, in chunks of 512. For a chunk, the row holding orig's content (src) moves to
// dst; a dst that is not itself a src has its content displaced, a src that is not a dst is
// freed; the k-th displaced row (by event order) moves into the k-th freed position. All
// source rows are read before any row is written, so swaps and cycles are safe. Freed hot
// positions lose residency: their KV slot no longer matches the Index row.
// The row <-> position maps are two identity arrays in global memory that the kernel puts
// back to identity before it returns, so nothing is re-initialised per round. Address and
// logical-id rows travel with their key row inside the chunk (the reference defers them to
// one commit; the service outputs were already published by the resolver, so the result is
// the same).
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kThreads = 1024;
constexpr uint32_t kChunk = 512;
constexpr uint32_t kSet = 2048;
constexpr uint32_t kEmpty = 0xffffffffu;
constexpr uint32_t kMaxPieces = 16;  // 16-byte pieces per key row (bf16 rows: 256 bytes)

__device__ __forceinline__ uint32_t set_hash(uint32_t k) { return (k * 0x9e3779b9u) >> 21; }
__device__ __forceinline__ bool set_insert(uint32_t* table, uint32_t k) {
  uint32_t h = set_hash(k);
  for (uint32_t i = 0; i < kSet; ++i) {
    const uint32_t old = atomicCAS(table + h, kEmpty, k);
    if (old == kEmpty) return true;
    if (old == k) return false;
    h = (h + 1u) & (kSet - 1u);
  }
  return false;
}
__device__ __forceinline__ bool set_contains(const uint32_t* table, uint32_t k) {
  uint32_t h = set_hash(k);
  for (uint32_t i = 0; i < kSet; ++i) {
    const uint32_t old = table[h];
    if (old == k) return true;
    if (old == kEmpty) return false;
    h = (h + 1u) & (kSet - 1u);
  }
  return false;
}

__global__ void __launch_bounds__(kThreads) exchange_rows(const KvipExchangeArgs a) {
  __shared__ uint32_t src_set[kSet], dst_set[kSet];
  __shared__ uint32_t plan_src[2 * kChunk], plan_dst[2 * kChunk];
  __shared__ uint32_t scan[33];
  __shared__ uint32_t error_word;
  const uint32_t b = blockIdx.x, tid = threadIdx.x, H = a.history, R = a.resident;
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  uint4* keys = reinterpret_cast<uint4*>(a.keys + static_cast<uint64_t>(owner) * H * a.key_row_bytes);
  float* scales = a.scales + static_cast<uint64_t>(owner) * H;
  int64_t* addresses = a.addresses + static_cast<uint64_t>(owner) * a.address_stride;
  int64_t* logical = a.logical_ids + static_cast<uint64_t>(owner) * H;
  int32_t* valid = a.hot_valid + static_cast<uint64_t>(owner) * R;
  uint32_t* row_pos = a.shadow + static_cast<uint64_t>(b) * 2u * H;  // original row -> position
  uint32_t* pos_row = row_pos + H;                                    // position -> original row
  const int32_t* ev_src = a.events_src + static_cast<uint64_t>(b) * kSlots;
  const int32_t* ev_dst = a.events_dst + static_cast<uint64_t>(b) * kSlots;
  const uint32_t pieces = a.key_row_bytes / 16u;
  if (tid == 0) error_word = a.row_status ? static_cast<uint32_t>(a.row_status[b * 32u]) : 0u;
  __syncthreads();

  uint32_t begin = 0;
  for (uint32_t q = 0; q < a.queries && !error_word; ++q) {
    const uint32_t count = static_cast<uint32_t>(a.query_counts[b * 8u + q]);
    for (uint32_t base = 0; base < count && !error_word; base += kChunk) {
      const uint32_t n = min(count - base, kChunk);
      for (uint32_t i = tid; i < kSet; i += kThreads) { src_set[i] = kEmpty; dst_set[i] = kEmpty; }
      __syncthreads();
      if (tid < n) {
        const uint32_t orig = static_cast<uint32_t>(ev_src[begin + base + tid]);
        const uint32_t dst = static_cast<uint32_t>(ev_dst[begin + base + tid]);
        const uint32_t src = orig < H ? row_pos[orig] : kEmpty;
        plan_src[tid] = src;
        plan_dst[tid] = dst;
        if (orig >= H || dst >= R || src >= H || !set_insert(src_set, src) || !set_insert(dst_set, dst))
          atomicOr(&error_word, 1u);
      }
      __syncthreads();
      if (error_word) break;
      const uint32_t displaced = tid < n && !set_contains(src_set, plan_dst[tid]) ? 1u : 0u;
      const uint32_t freed = tid < n && !set_contains(dst_set, plan_src[tid]) ? 1u : 0u;
      uint32_t totals;
      const uint32_t paired = block_exclusive_scan(displaced | (freed << 16), scan, &totals);
      if (displaced) plan_src[kChunk + (paired & 0xffffu)] = plan_dst[tid];
      if (freed) plan_dst[kChunk + (paired >> 16)] = plan_src[tid];
      __syncthreads();
      const uint32_t extras = totals & 0xffffu, moves = n + extras;
      auto move_index = [&](uint32_t i) { return i < n ? i : kChunk + i - n; };
      // snapshot every source row, then write
      uint4 piece[kMaxPieces];
      const uint32_t total_pieces = moves * pieces;
#pragma unroll
      for (uint32_t k = 0; k < kMaxPieces; ++k) {
        const uint32_t x = k * kThreads + tid;
        if (x < total_pieces) piece[k] = keys[static_cast<uint64_t>(plan_src[move_index(x / pieces)]) * pieces + x % pieces];
      }
      float scale_v = 0.f;
      int64_t address_v = 0, logical_v = 0;
      uint32_t row_v = 0;
      if (tid < moves) {
        const uint32_t s = plan_src[move_index(tid)];
        scale_v = scales[s]; address_v = addresses[s]; logical_v = logical[s]; row_v = pos_row[s];
      }
      __syncthreads();
#pragma unroll
      for (uint32_t k = 0; k < kMaxPieces; ++k) {
        const uint32_t x = k * kThreads + tid;
        if (x < total_pieces) keys[static_cast<uint64_t>(plan_dst[move_index(x / pieces)]) * pieces + x % pieces] = piece[k];
      }
      if (tid < moves) {
        const uint32_t d = plan_dst[move_index(tid)];
        scales[d] = scale_v; addresses[d] = address_v; logical[d] = logical_v;
        pos_row[d] = row_v;
        row_pos[row_v] = d;
        if (tid >= n && d < R) valid[d] = 0;  // closure destination: KV did not move with the row
      }
      __threadfence_block();
      __syncthreads();
    }
    begin += count;

  }
  __syncthreads();
  // put the maps back to identity for every position an event can have touched
  uint32_t all_events = 0;
  for (uint32_t q = 0; q < a.queries; ++q) all_events += static_cast<uint32_t>(a.query_counts[b * 8u + q]);
  for (uint32_t i = tid; i < all_events; i += kThreads) {
    const uint32_t orig = static_cast<uint32_t>(ev_src[i]), dst = static_cast<uint32_t>(ev_dst[i]);
    if (orig < H) { row_pos[orig] = orig; pos_row[orig] = orig; }
    if (dst < H) { row_pos[dst] = dst; pos_row[dst] = dst; }
  }

  if (error_word) {  // a failed owner loses hot residency (index_cache_update.h:6-20)
    for (uint32_t s = tid; s < R; s += kThreads) valid[s] = 0;
  }
  if (tid == 0) a.status[b] = static_cast<int32_t>(error_word);
}

}  // namespace

uint32_t launch_exchange(const KvipExchangeArgs& a, cudaStream_t stream) {
  exchange_rows<<<a.batch, kThreads, 0, stream>>>(a);
  count_launch();
  return check_launch("exchange_rows");
}

}  // namespace kvip

extern "C" uint32_t kvip_b200_exchange(const KvipExchangeArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->keys && a->scales && a->addresses && a->logical_ids && a->hot_valid && a->events_src &&
                   a->events_dst && a->query_counts && a->shadow && a->status, "exchange: null pointer");
  KVIP_REQUIRE(a->batch >= 1 && a->queries >= 1 && a->queries <= KVIP_MAX_QUERIES, "exchange: bad batch/queries");
  KVIP_REQUIRE(a->key_row_bytes == 128 || a->key_row_bytes == 256, "exchange: key rows are 128 or 256 bytes");
  KVIP_REQUIRE(a->resident <= a->history && a->address_stride >= a->history, "exchange: geometry");
  KVIP_REQUIRE((reinterpret_cast<uintptr_t>(a->keys) & 15u) == 0, "exchange: keys must be 16-byte aligned");
  return kvip::launch_exchange(*a, static_cast<cudaStream_t>(stream));
}
