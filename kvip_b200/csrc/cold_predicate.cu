// Resident threshold and cold predicate: which non-resident tokens can still reach the final TopK.
//
// The reference first selects the TopK of the RESIDENT prefix of a score row (positions below `resident`,
// ProcessResidentTopK, op_kernel/indexer/indexer_vector.h:100-105), keeps the smallest selected key as the
// row's threshold (SaveResident, :162-177) and then marks every cold position whose score beats it
// (ClassifyScore / BatchClassifyScore, indexer_score.h:784-792, 976-1017): only those can displace a
// resident winner, so they are the candidates of the speculative prefetch. Adding positions to a row can only
// raise its 2048th largest key, so the marked set always contains the cold part of the final TopK.
//
// Here the prefix TopK is the ordinary TopK kernel run with every row's query end clipped to `resident`; this
// kernel takes its output, derives the threshold, and streams the cold part of the row once: one bit per
// position, 32 positions per word (warp ballots), plus the number of marked positions per row.
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kThreads = 1024;

__global__ void __launch_bounds__(kThreads) cold_predicate(const KvipColdArgs a) {
  __shared__ uint32_t reduce[32];
  __shared__ uint32_t shared_threshold;
  const uint32_t row = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint32_t b = row / a.queries;
  int32_t valid_len = min(a.key_lengths[b], a.query_ends[row]);
  valid_len = min(valid_len, static_cast<int32_t>(a.scoreStride));
  const uint32_t L = valid_len > 0 ? static_cast<uint32_t>(valid_len) : 0u;
  const float* scores = a.scores + static_cast<uint64_t>(row) * a.scoreStride;
  // threshold key: the smallest key of the prefix TopK, or 0 (everything beats it) while the resident prefix
  // holds fewer than 2048 valid positions
  uint32_t smallest = 0xffffffffu;
  bool full = true;
  for (uint32_t i = tid; i < kTop; i += kThreads) {
    const int32_t position = a.prefix_topk[static_cast<uint64_t>(row) * kTop + i];
    if (position < 0) full = false;
    else smallest = min(smallest, sortable_key(a.prefix_scores[static_cast<uint64_t>(row) * kTop + i]));
  }
  smallest = full ? smallest : 0u;
#pragma unroll
  for (uint32_t d = 16; d > 0; d >>= 1) smallest = min(smallest, __shfl_xor_sync(0xffffffffu, smallest, d));
  if (lane == 0) reduce[warp] = smallest;
  __syncthreads();
  if (warp == 0) {
    uint32_t v = reduce[lane];
#pragma unroll
    for (uint32_t d = 16; d > 0; d >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, d));
    if (lane == 0) shared_threshold = v;
  }
  __syncthreads();
  const uint32_t threshold = shared_threshold;
  if (tid == 0) a.threshold_keys[row] = threshold;
  // cold part of the row: word w covers positions resident + 32 w .. + 31
  const uint32_t words = a.bitmap_words;
  uint32_t* bitmap = a.bitmap + static_cast<uint64_t>(row) * words;
  uint32_t marked = 0;
  for (uint32_t w0 = 0; w0 < words; w0 += kThreads / 32u) {   // every warp: the same trip count
    const uint32_t w = w0 + warp;
    const uint32_t position = a.resident + w * 32u + lane;
    const bool live = w < words && position < L;
    const float x = live ? scores[position] : 0.f;
    const uint32_t bits = __ballot_sync(0xffffffffu, live && sortable_key(x) > threshold);
    if (lane == 0 && w < words) bitmap[w] = bits;
    marked += lane == 0 ? __popc(bits) : 0u;
  }
  __syncthreads();
  if (lane == 0) reduce[warp] = marked;
  __syncthreads();
  if (warp == 0) {
    uint32_t v = reduce[lane];
#pragma unroll
    for (uint32_t d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    if (lane == 0) a.counts[row] = static_cast<int32_t>(v);
  }
}

}  // namespace
}  // namespace kvip

extern "C" uint32_t kvip_b200_cold_predicate(const KvipColdArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->scores && a->key_lengths && a->query_ends && a->prefix_topk && a->prefix_scores &&
                   a->threshold_keys && a->bitmap && a->counts, "cold_predicate: null pointer");
  KVIP_REQUIRE(a->rows >= 1 && a->queries >= 1 && a->rows % a->queries == 0, "cold_predicate: rows must be batch*queries");
  KVIP_REQUIRE(a->resident % 32u == 0 && a->resident <= a->scoreStride, "cold_predicate: resident must be a multiple of 32 inside the row");
  KVIP_REQUIRE(static_cast<uint64_t>(a->bitmap_words) * 32u >= a->scoreStride - a->resident,
               "cold_predicate: the bitmap does not cover the cold part of a row");
  kvip::cold_predicate<<<a->rows, kvip::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("cold_predicate");
}
