// Per-query TopK-2048 by radix select over fp32 scores, and the merge of sequence-sharded
// candidates.
//
// Contract (the reference kernel's order, op_kernel/indexer/topk_common.h:1136-1187 and
// indexer_vector.h:826-957, stated over the whole row): with L valid positions,
//   L <= 0      -> 2048 x -1
//   L <= 2048   -> 0, 1, ..., L-1, then -1
//   otherwise   -> v = 2048th largest key; every position with key > v in ascending
//                  position, then positions with key == v in ascending position, cut at 2048.
// Ties therefore go to the lower token index, and the output is a deterministic function
// of the score row.
//
// topk_select: one CTA per query row. Three histogram passes (12 + 12 + 8 bits of the order-preserving
// u32 image of the float) find v exactly; a fourth, ordered pass compacts the winners with
// block-wide prefix sums (no atomics, so the order is the position order). The row is read
// from L2 (the LI kernel has just written it) with 16-byte loads.
#include <cooperative_groups.h>
#include "common.cuh"
#include "topk_core.cuh"

namespace kvip {
namespace {

using namespace topk_core;

// First radix pass spread over the whole GPU: `segments` CTAs per row add their slice's 12-bit
// histogram to the row's histogram in global memory (the selecting CTA clears it again after use).
constexpr uint32_t kHistThreads = 256;

__global__ void __launch_bounds__(kHistThreads) topk_histogram(const KvipTopkArgs a) {
  __shared__ uint32_t hist[4096];
  const uint32_t row = blockIdx.y, tid = threadIdx.x;
  int32_t valid_len = min(a.key_lengths[row / a.queries], a.query_ends[row]);
  valid_len = min(valid_len, static_cast<int32_t>(a.scoreStride));
  if (valid_len <= static_cast<int32_t>(kTop)) return;
  const uint32_t L = static_cast<uint32_t>(valid_len), vec_count = (L + 3u) >> 2;
  const uint32_t per = ((vec_count + gridDim.x - 1u) / gridDim.x + kHistThreads - 1u) / kHistThreads * kHistThreads;
  const uint32_t begin = blockIdx.x * per, end = min(begin + per, vec_count);
  if (begin >= end) return;
  for (uint32_t i = tid; i < 4096; i += kHistThreads) hist[i] = 0;
  __syncthreads();
  const float4* row4 = reinterpret_cast<const float4*>(a.scores + static_cast<uint64_t>(row) * a.scoreStride);
  for (uint32_t v0 = begin; v0 < end; v0 += kHistThreads) {  // `per` is a multiple of the block: warps stay converged
    const uint32_t v = v0 + tid;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (v < end) x = row4[v];
    const float e[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j)
      hist_add(hist, v < end && (v * 4u + j) < L, sortable_key(e[j]) >> 20);
  }
  __syncthreads();
  uint32_t* out = a.histogram + static_cast<uint64_t>(row) * 4096u;
  for (uint32_t i = tid; i < 4096; i += kHistThreads)
    if (hist[i]) atomicAdd(out + i, hist[i]);
}

__global__ void __launch_bounds__(kThreads) topk_select(const KvipTopkArgs a) {
  select_row(a, blockIdx.x, a.histogram + static_cast<uint64_t>(blockIdx.x) * 4096u);
}

// ---- merge of shard candidates -----------------------------------------------------------
// One CTA per row. The candidates (shards x 2048 (score, index) pairs, at most 16384) are loaded into shared
// memory once; the 2048th largest key is found by radix select over them (three passes over shared memory), ties
// at that key are settled towards the lower index by a second radix select over the tied indices, the 2048
// winners are compacted and only they are sorted (by "is a tie", then index): the canonical order. Sorting all
// candidates instead cost 105 block-wide compare-exchange rounds over 16384 entries; this takes 66 over 2048, of
// which only the 15 with a partner distance of 64 or more go through shared memory and a block barrier.
constexpr uint32_t kMergeMax = 8u * kTop;

// Ascending bitonic sort of data[0..2048) by the 1024 threads of the block. Thread t keeps elements 2t and 2t+1 in
// registers, so a warp owns 64 consecutive elements: compare-exchange rounds with a partner distance below 64 are
// register moves and warp shuffles, the others work on shared memory between block barriers.
__device__ __forceinline__ void bitonic_sort_2048(uint32_t* data) {
  const uint32_t t = threadIdx.x, e0 = 2u * t;
  uint32_t x0 = data[e0], x1 = data[e0 + 1u];
  auto in_warp = [&](uint32_t k, uint32_t j_from) {   // rounds j_from, j_from / 2, ..., 1 of merge width k
    const bool ascending = (e0 & k) == 0;
    for (uint32_t j = j_from; j >= 2u; j >>= 1) {
      const bool keep_min = ((e0 & j) == 0) == ascending;
      const uint32_t y0 = __shfl_xor_sync(0xffffffffu, x0, j >> 1), y1 = __shfl_xor_sync(0xffffffffu, x1, j >> 1);
      x0 = keep_min ? min(x0, y0) : max(x0, y0);
      x1 = keep_min ? min(x1, y1) : max(x1, y1);
    }
    const uint32_t low = min(x0, x1), high = max(x0, x1);
    x0 = ascending ? low : high;
    x1 = ascending ? high : low;
  };
  for (uint32_t k = 2; k <= 64u; k <<= 1) in_warp(k, k >> 1);
  for (uint32_t k = 128; k <= kTop; k <<= 1) {
    data[e0] = x0;
    data[e0 + 1u] = x1;
    __syncthreads();
    for (uint32_t j = k >> 1; j >= 64u; j >>= 1) {
      const uint32_t e = (t / j) * (2u * j) + (t % j);   // the lower element of this thread's pair
      const uint32_t x = data[e], y = data[e + j];
      if ((x > y) == ((e & k) == 0)) { data[e] = y; data[e + j] = x; }
      __syncthreads();
    }
    x0 = data[e0];
    x1 = data[e0 + 1u];
    in_warp(k, 32u);
  }
  data[e0] = x0;
  data[e0 + 1u] = x1;
  __syncthreads();
}

// Histogram add for candidates that mostly share their leading digits (the best scores of every shard lie close
// together): lanes with the same bin are found with a match vote and one of them adds for all, so a warp issues one
// shared-memory atomic per DISTINCT bin instead of up to 32 serialised ones on the same word.
__device__ __forceinline__ void hist_add_matched(uint32_t* hist, bool valid, uint32_t bin) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (valid) {
    const uint32_t peers = __match_any_sync(active, bin);
    if ((threadIdx.x & 31u) == static_cast<uint32_t>(__ffs(static_cast<int>(peers)) - 1)) atomicAdd(hist + bin, __popc(peers));
  }
}

// The `want`-th largest of the values value(i), i < n with member(i) (12 + 12 + 8 bit radix select, all threads of
// the block call). Returns the value; *take = how many entries EQUAL to it belong to the `want` largest, *equal = how
// many entries equal it in all.
template <typename Value, typename Member>
__device__ uint32_t kth_largest(uint32_t n, uint32_t want, Value value, Member member, uint32_t* hist, uint32_t* scan_scratch,
                                uint32_t* found, uint32_t* take, uint32_t* equal) {
  const uint32_t tid = threadIdx.x;
  uint32_t prefix = 0, prefix_mask = 0, remaining = want;
#pragma unroll 1
  for (uint32_t pass = 0; pass < 3; ++pass) {
    const uint32_t bits = pass == 2 ? 8u : 12u;
    const uint32_t shift = pass == 0 ? 20u : (pass == 1 ? 8u : 0u);
    const uint32_t bins = 1u << bits;
    for (uint32_t i = tid; i < bins; i += kThreads) hist[i] = 0;
    if (tid == 0) { found[0] = 0; found[1] = 0; found[2] = 0; }
    __syncthreads();
    for (uint32_t r = 0; r * kThreads < n; ++r) {   // block-uniform trip count: the add votes per warp
      const uint32_t i = r * kThreads + tid;
      const bool in = i < n && member(i);
      const uint32_t v = in ? value(i) : 0u;
      hist_add_matched(hist, in && (v & prefix_mask) == prefix, (v >> shift) & (bins - 1u));
    }
    __syncthreads();
    const uint32_t per = bins / kThreads ? bins / kThreads : 1u;  // 4, 4, then 1 (256 bins)
    const uint32_t groups = bins / per;
    const uint32_t group = groups - 1u - tid;  // valid when tid < groups: the highest bins first
    uint32_t local = 0;
    if (tid < groups)
      for (uint32_t j = 0; j < per; ++j) local += hist[group * per + j];
    uint32_t above = block_exclusive_scan(local, scan_scratch, nullptr);
    if (tid < groups) {
      for (int32_t j = static_cast<int32_t>(per) - 1; j >= 0; --j) {
        const uint32_t count = hist[group * per + static_cast<uint32_t>(j)];
        if (above < remaining && above + count >= remaining) {
          found[0] = group * per + static_cast<uint32_t>(j);
          found[1] = remaining - above;
          found[2] = count;
        }
        above += count;
      }
    }
    __syncthreads();
    prefix |= found[0] << shift;
    prefix_mask |= (bins - 1u) << shift;
    remaining = found[1];
    *equal = found[2];   // of the last pass: the entries that match in every digit
    __syncthreads();
  }
  *take = remaining;
  return prefix;
}

__global__ void __launch_bounds__(kThreads) topk_merge(const KvipMergeArgs a) {
  extern __shared__ uint32_t merge_smem[];   // [n] keys, [n] indices, [2048] winners
  __shared__ uint32_t hist[4096];
  __shared__ uint32_t scan_scratch[33];
  __shared__ uint32_t found[3];
  const uint32_t row = blockIdx.x, tid = threadIdx.x, n = a.shards * kTop;
  const float* cand_scores = a.cand_scores;
  const int32_t* cand_index = a.cand_index;
  if (a.peer_block) {
    // Candidates delivered by peer_exchange: wait until every rank's flag in this rank's exchange block has reached the
    // block's step counter (this rank's own exchange kernel, earlier on this stream, set the counter and its own flag;
    // the other flags are written from other GPUs). The wait is bounded; when it runs out the rows come back as -1.
    __shared__ uint32_t gave_up;
    const uint8_t* block = static_cast<const uint8_t*>(a.peer_block);
    const uint32_t step = *reinterpret_cast<const volatile uint32_t*>(block);
    if (tid == 0) gave_up = 0;
    __syncthreads();
    if (tid < a.wait_ranks) {
      const volatile uint32_t* flag = reinterpret_cast<const volatile uint32_t*>(block + 256) + tid;
      const long long limit = static_cast<long long>(a.wait_kilocycles ? a.wait_kilocycles : 2000000u) << 10;
      const long long start = clock64();
      // flags only grow, and a later step overwrites the other half of the block: "reached" is >=, compared as a
      // signed difference so that the counter may wrap
      while (static_cast<int32_t>(*flag - step) < 0) {
        if (clock64() - start > limit) { gave_up = 1u; break; }
      }
    }
    __threadfence_system();   // the candidates behind a flag are read after the flag
    __syncthreads();
    if (gave_up) {
      if (tid == 0 && a.status) atomicOr(a.status, static_cast<int32_t>(KVIP_ERR_PEER));
      for (uint32_t i = tid; i < kTop; i += kThreads) a.topk[static_cast<uint64_t>(row) * kTop + i] = -1;
      return;   // block-uniform
    }
    const uint64_t block_bytes = static_cast<uint64_t>(a.rows) * 2u * kTop * 4u;
    const int32_t* half = reinterpret_cast<const int32_t*>(block + KVIP_PEER_HEADER_BYTES +
                                                           static_cast<uint64_t>(step & 1u) * a.shards * block_bytes);
    cand_scores = reinterpret_cast<const float*>(half);
    cand_index = half + static_cast<uint64_t>(a.rows) * kTop;
  }
  uint32_t* keys = merge_smem;
  int32_t* index = reinterpret_cast<int32_t*>(merge_smem + n);
  uint32_t* winners = merge_smem + 2u * n;
  const uint64_t shard_stride = a.shard_stride ? a.shard_stride : kTop;
  const uint64_t row_offset = static_cast<uint64_t>(row) * (a.row_stride ? a.row_stride : n);
  uint32_t mine = 0;
  for (uint32_t i = tid; i < n; i += kThreads) {
    const uint64_t at = row_offset + (i / kTop) * shard_stride + (i % kTop);
    const int32_t candidate = __ldcg(cand_index + at);   // L2 loads: the lists may have been written by another GPU
    index[i] = candidate;
    keys[i] = candidate >= 0 ? sortable_key(__ldcg(cand_scores + at)) : 0u;
    mine += candidate >= 0 ? 1u : 0u;
  }
  uint32_t valid;
  block_exclusive_scan(mine, scan_scratch, &valid);   // also the barrier after the loads
  // the cut: key of the 2048th largest candidate, how many candidates tied at it are taken, and below which index
  uint32_t cut_key = 0, ties_taken = 0, tie_index_limit = 0xffffffffu;   // defaults: every valid candidate wins
  if (valid > kTop) {   // block-uniform
    uint32_t tied = 0;
    cut_key = kth_largest(n, kTop, [&](uint32_t i) { return keys[i]; }, [&](uint32_t i) { return index[i] >= 0; }, hist,
                          scan_scratch, found, &ties_taken, &tied);
    if (ties_taken < tied) {   // block-uniform; with distinct scores at the cut there is nothing to settle
      // lower index first among the tied: the ties_taken smallest indices = the ties_taken largest of ~index
      uint32_t unused, unused_too;
      const uint32_t inverted = kth_largest(n, ties_taken, [&](uint32_t i) { return ~static_cast<uint32_t>(index[i]); },
                                            [&](uint32_t i) { return index[i] >= 0 && keys[i] == cut_key; }, hist,
                                            scan_scratch, found, &unused, &unused_too);
      tie_index_limit = ~inverted;   // indices are distinct: exactly ties_taken tied candidates lie at or below it
    }
  }
  // winners, compacted in input order (a thread owns a contiguous run of candidates), as (is a tie, index). With a
  // cut they are then sorted: keys above the cut by ascending index, the tied ones after them by ascending index.
  // Without a cut (at most 2048 valid candidates) the input order IS the canonical one and is kept: the shards are in
  // position order and each shard's list is canonical for its slice - ascending positions for a slice of at most
  // 2048 keys, the whole answer when one shard alone contributes.
  for (uint32_t i = tid; i < kTop; i += kThreads) winners[i] = 0xffffffffu;
  __syncthreads();
  auto classify = [&](uint32_t i, bool* tie) -> bool {
    if (index[i] < 0) return false;
    *tie = valid > kTop && keys[i] == cut_key;
    return valid <= kTop || keys[i] > cut_key || (*tie && static_cast<uint32_t>(index[i]) <= tie_index_limit);
  };
  const uint32_t per = n / kThreads;   // n is a multiple of 2048
  uint32_t won = 0;
  bool tie = false;
  for (uint32_t i = tid * per; i < (tid + 1u) * per; ++i) won += classify(i, &tie) ? 1u : 0u;
  uint32_t at = block_exclusive_scan(won, scan_scratch, nullptr);
  for (uint32_t i = tid * per; i < (tid + 1u) * per; ++i)
    if (classify(i, &tie)) {
      if (at < kTop) winners[at] = (tie ? 0x80000000u : 0u) | static_cast<uint32_t>(index[i]);
      ++at;
    }
  __syncthreads();
  if (valid > kTop) bitonic_sort_2048(winners);   // block-uniform
  int32_t* out = a.topk + static_cast<uint64_t>(row) * kTop;
  for (uint32_t i = tid; i < kTop; i += kThreads)
    out[i] = winners[i] == 0xffffffffu ? -1 : static_cast<int32_t>(winners[i] & 0x7fffffffu);
}

// ---- merge of shard candidates on a cluster: one CTA per shard --------------------------------------------------
// The single-CTA merge above walks shards x 2048 candidates with 1024 threads (16 rounds per radix pass at eight
// shards) and measured 66 us there, more than the score pass and the local TopK of the same step together. Here a
// cluster of `shards` CTAs shares the work: CTA c owns shard c's 2048 candidates, two per thread, in registers. The
// hub (cluster rank 0) owns the histograms, the digit found per pass and the winners' list; the others reach them
// through distributed shared memory. Per radix pass: every CTA histograms its candidates locally and adds its
// non-empty bins to the hub's histogram, cluster barrier, the hub scans, cluster barrier, everyone reads the digit.
// Same result as topk_merge, bit for bit (same cut, same tie rule, same canonical order).
struct MergeHub {
  uint32_t hist[2][4096];   // double-buffered: the hub clears the next pass's copy while it scans this one's
  uint32_t winners[kTop];
  uint32_t valid[8], won[8], bad[8];
  uint32_t found[3];        // digit, how many of the wanted still lie in that bin, entries in that bin
};

namespace cg = cooperative_groups;

__global__ void __launch_bounds__(kThreads, 1) topk_merge_cluster(const KvipMergeArgs a) {
  extern __shared__ __align__(16) uint8_t hub_raw[];   // one MergeHub; used on rank 0 only (same image in every CTA)
  MergeHub& hub_here = *reinterpret_cast<MergeHub*>(hub_raw);
  __shared__ uint32_t local_hist[4096];
  __shared__ uint32_t scan_scratch[33];
  __shared__ uint32_t shared_word[4];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t shards = a.shards, shard = cluster.block_rank(), row = blockIdx.x / shards, tid = threadIdx.x;
  MergeHub* hub = cluster.map_shared_rank(&hub_here, 0);

  const float* cand_scores = a.cand_scores;
  const int32_t* cand_index = a.cand_index;
  uint32_t gave_up = 0;
  if (a.peer_block) {   // CTA c waits for rank c's flag only
    const uint8_t* block = static_cast<const uint8_t*>(a.peer_block);
    const uint32_t step = *reinterpret_cast<const volatile uint32_t*>(block);
    if (tid == 0) {
      const volatile uint32_t* flag = reinterpret_cast<const volatile uint32_t*>(block + 256) + shard;
      const long long limit = static_cast<long long>(a.wait_kilocycles ? a.wait_kilocycles : 2000000u) << 10;
      const long long start = clock64();
      uint32_t failed = 0;
      while (static_cast<int32_t>(*flag - step) < 0) {
        if (clock64() - start > limit) { failed = 1u; break; }
      }
      shared_word[0] = failed;
    }
    __threadfence_system();
    __syncthreads();
    gave_up = shared_word[0];
    const uint64_t block_bytes = static_cast<uint64_t>(a.rows) * 2u * kTop * 4u;
    const int32_t* half = reinterpret_cast<const int32_t*>(block + KVIP_PEER_HEADER_BYTES +
                                                           static_cast<uint64_t>(step & 1u) * shards * block_bytes);
    cand_scores = reinterpret_cast<const float*>(half);
    cand_index = half + static_cast<uint64_t>(a.rows) * kTop;
  }
  // two consecutive candidates per thread: a thread's pair, and the threads in order, keep the input order
  const uint64_t shard_stride = a.shard_stride ? a.shard_stride : kTop;
  const uint64_t at = static_cast<uint64_t>(row) * (a.row_stride ? a.row_stride : shards * kTop) + shard * shard_stride + 2u * tid;
  int32_t index[2] = {-1, -1};
  uint32_t key[2] = {0u, 0u};
  if (!gave_up) {
    const int2 two_index = __ldcg(reinterpret_cast<const int2*>(cand_index + at));       // L2 loads: another GPU may
    const float2 two_score = __ldcg(reinterpret_cast<const float2*>(cand_scores + at));  // have written the lists
    index[0] = two_index.x; index[1] = two_index.y;
    key[0] = index[0] >= 0 ? sortable_key(two_score.x) : 0u;
    key[1] = index[1] >= 0 ? sortable_key(two_score.y) : 0u;
  }
  uint32_t valid_here;
  const uint32_t valid_before = block_exclusive_scan((index[0] >= 0 ? 1u : 0u) + (index[1] >= 0 ? 1u : 0u), scan_scratch, &valid_here);
  if (shard == 0)
    for (uint32_t i = tid; i < 2u * 4096u; i += kThreads) hub_here.hist[0][i] = 0;
  if (tid == 0) { hub->valid[shard] = valid_here; hub->bad[shard] = gave_up; }
  cluster.sync();
  // every CTA learns all counts (and whether any wait ran out): thread r reads entry r of the hub
  if (tid < shards) { local_hist[tid] = hub->valid[tid]; local_hist[8 + tid] = hub->bad[tid]; }
  __syncthreads();
  uint32_t total_valid = 0, before_me = 0, any_bad = 0;
  for (uint32_t r = 0; r < shards; ++r) {
    if (r < shard) before_me += local_hist[r];
    total_valid += local_hist[r];
    any_bad |= local_hist[8 + r];
  }
  __syncthreads();   // local_hist is reused below: as the per-CTA histogram, all zero between passes
  for (uint32_t i = tid; i < 4096u; i += kThreads) local_hist[i] = 0;
  __syncthreads();
  int32_t* out = a.topk + static_cast<uint64_t>(row) * kTop;
  // A CTA that leaves here must not do so while another one may still be reading the hub's counts: one more cluster
  // barrier on the two early ways out (both are cluster-uniform decisions).
  if (any_bad) {
    cluster.sync();
    if (shard == 0) {
      if (tid == 0 && a.status) atomicOr(a.status, static_cast<int32_t>(KVIP_ERR_PEER));
      for (uint32_t i = tid; i < kTop; i += kThreads) out[i] = -1;
    }
    return;
  }
  if (total_valid <= kTop) {   // nothing is cut, the input order is the canonical one
    cluster.sync();
    uint32_t w = before_me + valid_before;
    if (index[0] >= 0) out[w++] = index[0];
    if (index[1] >= 0) out[w++] = index[1];
    if (shard == 0)
      for (uint32_t i = total_valid + tid; i < kTop; i += kThreads) out[i] = -1;
    return;
  }

  // cluster-wide "want-th largest" of value(j) over the members, j = 0, 1 the thread's two candidates
  uint32_t select_calls = 0;
  auto kth_largest_cluster = [&](uint32_t want, const uint32_t (&value)[2], const bool (&member)[2], uint32_t* take,
                                 uint32_t* equal) -> uint32_t {
    uint32_t prefix = 0, prefix_mask = 0, remaining = want;
#pragma unroll 1
    for (uint32_t pass = 0; pass < 3; ++pass) {
      const uint32_t bits = pass == 2 ? 8u : 12u;
      const uint32_t shift = pass == 0 ? 20u : (pass == 1 ? 8u : 0u);
      const uint32_t bins = 1u << bits;
      const uint32_t buffer = (select_calls * 3u + pass) & 1u;   // the hub's histogram of this pass (cleared already)
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j)   // local_hist is all zero here: cleared below as it is flushed
        hist_add_matched(local_hist, member[j] && (value[j] & prefix_mask) == prefix, (value[j] >> shift) & (bins - 1u));
      __syncthreads();
      for (uint32_t i = tid; i < bins; i += kThreads) {
        const uint32_t count = local_hist[i];
        if (count) {
          atomicAdd(&hub->hist[buffer][i], count);
          local_hist[i] = 0;
        }
      }
      cluster.sync();   // also the block barrier between clearing local_hist and the next pass's adds
      if (shard == 0) {
        uint32_t* hist = hub_here.hist[buffer];
        uint32_t* next = hub_here.hist[buffer ^ 1u];
        for (uint32_t i = tid; i < 4096u; i += kThreads) next[i] = 0;   // nobody adds to it before the next barrier
        const uint32_t per = bins / kThreads ? bins / kThreads : 1u;
        const uint32_t groups = bins / per;
        const uint32_t group = groups - 1u - tid;   // valid when tid < groups: the highest bins first
        uint32_t local = 0;
        if (tid < groups)
          for (uint32_t j = 0; j < per; ++j) local += hist[group * per + j];
        if (tid == 0) { hub_here.found[0] = 0; hub_here.found[1] = 0; hub_here.found[2] = 0; }
        uint32_t above = block_exclusive_scan(local, scan_scratch, nullptr);   // also orders the reset before the writes
        if (tid < groups) {
          for (int32_t j = static_cast<int32_t>(per) - 1; j >= 0; --j) {
            const uint32_t count = hist[group * per + static_cast<uint32_t>(j)];
            if (above < remaining && above + count >= remaining) {
              hub_here.found[0] = group * per + static_cast<uint32_t>(j);
              hub_here.found[1] = remaining - above;
              hub_here.found[2] = count;
            }
            above += count;
          }
        }
      }
      cluster.sync();
      // every thread reads the three words from the hub (warp-uniform addresses); the hub rewrites them only after
      // the next cluster barrier
      prefix |= hub->found[0] << shift;
      prefix_mask |= (bins - 1u) << shift;
      remaining = hub->found[1];
      *equal = hub->found[2];
    }
    ++select_calls;
    *take = remaining;
    return prefix;
  };

  const bool is_valid[2] = {index[0] >= 0, index[1] >= 0};
  uint32_t ties_taken = 0, tied = 0, tie_index_limit = 0xffffffffu;
  const uint32_t cut_key = kth_largest_cluster(kTop, key, is_valid, &ties_taken, &tied);
  if (ties_taken < tied) {   // cluster-uniform: some candidates tied at the cut are left out: the lower indices win
    const uint32_t inverted_index[2] = {~static_cast<uint32_t>(index[0]), ~static_cast<uint32_t>(index[1])};
    const bool is_tied[2] = {is_valid[0] && key[0] == cut_key, is_valid[1] && key[1] == cut_key};
    uint32_t unused, unused_too;
    tie_index_limit = ~kth_largest_cluster(ties_taken, inverted_index, is_tied, &unused, &unused_too);
  }
  // winners, compacted in input order into the hub's list as (is a tie, index); the hub sorts and writes them
  bool wins[2], tie[2];
#pragma unroll
  for (uint32_t j = 0; j < 2; ++j) {
    tie[j] = is_valid[j] && key[j] == cut_key;
    wins[j] = is_valid[j] && (key[j] > cut_key || (tie[j] && static_cast<uint32_t>(index[j]) <= tie_index_limit));
  }
  uint32_t won_here;
  const uint32_t won_before = block_exclusive_scan((wins[0] ? 1u : 0u) + (wins[1] ? 1u : 0u), scan_scratch, &won_here);
  if (tid == 0) hub->won[shard] = won_here;
  if (shard == 0)
    for (uint32_t i = tid; i < kTop; i += kThreads) hub_here.winners[i] = 0xffffffffu;
  cluster.sync();
  if (tid < shards) local_hist[tid] = hub->won[tid];
  __syncthreads();
  uint32_t w = won_before;
  for (uint32_t r = 0; r < shard; ++r) w += local_hist[r];
#pragma unroll
  for (uint32_t j = 0; j < 2; ++j)
    if (wins[j]) {
      if (w < kTop) hub->winners[w] = (tie[j] ? 0x80000000u : 0u) | static_cast<uint32_t>(index[j]);
      ++w;
    }
  cluster.sync();
  if (shard != 0) return;
  bitonic_sort_2048(hub_here.winners);
  for (uint32_t i = tid; i < kTop; i += kThreads)
    out[i] = hub_here.winners[i] == 0xffffffffu ? -1 : static_cast<int32_t>(hub_here.winners[i] & 0x7fffffffu);
}

}  // namespace

uint32_t launch_topk_split(const KvipTopkArgs& a, cudaStream_t stream);
uint32_t launch_topk_pivot(const KvipTopkArgs& a, cudaStream_t stream);

// Path by what the caller supplies: no scratch -> one CTA per row, sampled pivot + one filtering pass over
// the row (topk_pivot.cu); `histogram` -> first radix pass spread over the GPU, then one CTA per row;
// `split_scratch` -> every pass spread over the GPU.
uint32_t launch_topk(const KvipTopkArgs& a, cudaStream_t stream) {
  if (a.split_scratch) return launch_topk_split(a, stream);
  if (!a.histogram) return launch_topk_pivot(a, stream);
  uint32_t segments = (4u * device_sm_count() + a.rows - 1u) / a.rows;
  segments = segments < 1u ? 1u : (segments > 32u ? 32u : segments);
  topk_histogram<<<dim3(segments, a.rows), kHistThreads, 0, stream>>>(a);
  count_launch();
  if (uint32_t bad = check_launch("topk_histogram")) return bad;
  // static + dynamic shared memory exceeds the 48 KiB default
  if (uint32_t bad = raise_dynamic_smem(kSlotTopkSelect, reinterpret_cast<const void*>(topk_select), 64 * 1024,
                                        "topk_select attribute"))
    return bad;
  topk_select<<<a.rows, kThreads, kCandidates * sizeof(uint32_t), stream>>>(a);
  count_launch();
  return check_launch("topk_select");
}

}  // namespace kvip

extern "C" uint32_t kvip_b200_topk(const KvipTopkArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->scores && a->key_lengths && a->query_ends && a->topk, "topk: null pointer");
  KVIP_REQUIRE(a->rows >= 1 && a->queries >= 1 && a->rows % a->queries == 0, "topk: rows must be batch*queries");
  KVIP_REQUIRE(a->scoreStride % 4 == 0 && (reinterpret_cast<uintptr_t>(a->scores) & 15u) == 0,
               "topk: score rows must be 16-byte aligned");
  return kvip::launch_topk(*a, static_cast<cudaStream_t>(stream));
}

// ---- TopK for callers that cannot allocate --------------------------------------------------------
// The split TopK needs a [rows, 4096] histogram scratch. Some hosts of this library have nowhere to get
// it from: a serving process that handed every free byte of HBM to its KV-cache pool at start-up (a later
// cudaMalloc fails or fragments the pool), or a decode-loop plugin that is forbidden to allocate because
// an allocation would stall the device it is feeding. For them the scratch lives in the library's own
// image: a fixed 4 MiB array that every GPU loading the library holds until the process exits.
#define KVIP_TOPK_STATIC_ROWS 256u
static __device__ __align__(256) uint32_t g_static_histogram[KVIP_TOPK_STATIC_ROWS * 4096u];

extern "C" uint32_t kvip_b200_topk_static(const KvipTopkArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->scores && a->key_lengths && a->query_ends && a->topk, "topk_static: null pointer");
  KVIP_REQUIRE(a->rows >= 1 && a->queries >= 1 && a->rows % a->queries == 0, "topk_static: rows must be batch*queries");
  KVIP_REQUIRE(a->rows <= KVIP_TOPK_STATIC_ROWS,
               "topk_static: more than 256 score rows do not fit the built-in scratch; split the call or use "
               "kvip_b200_topk with a caller-provided histogram");
  KVIP_REQUIRE(a->scoreStride % 4 == 0 && (reinterpret_cast<uintptr_t>(a->scores) & 15u) == 0,
               "topk_static: score rows must be 16-byte aligned");
  // In host code `g_static_histogram` is only a stand-in for the symbol; the address kernels can use is
  // looked up once per device, with that device current.
  constexpr int kMaxDevices = 64;
  static uint32_t* scratch_of_device[kMaxDevices] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return kvip::check_launch("topk_static: cudaGetDevice");
  if (!scratch_of_device[device]) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_static_histogram) != cudaSuccess || !address)
      return kvip::check_launch("topk_static: cudaGetSymbolAddress");
    scratch_of_device[device] = static_cast<uint32_t*>(address);
  }
  uint32_t* scratch = scratch_of_device[device];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // every call shares the array and finds what the last call left: the rows used now must start at zero
  if (cudaMemsetAsync(scratch, 0, static_cast<size_t>(a->rows) * 4096u * sizeof(uint32_t), s) != cudaSuccess)
    return kvip::check_launch("topk_static: clearing the scratch");
  KvipTopkArgs with_scratch = *a;
  with_scratch.histogram = scratch;
  with_scratch.split_scratch = nullptr;
  return kvip::launch_topk(with_scratch, s);
}

extern "C" uint32_t kvip_b200_topk_merge(const KvipMergeArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->topk && ((a->cand_scores && a->cand_index) || a->peer_block), "topk_merge: null pointer");
  KVIP_REQUIRE(!a->peer_block || (a->wait_ranks == a->shards && (reinterpret_cast<uintptr_t>(a->peer_block) & 255) == 0),
               "topk_merge: a peer exchange block is waited for by all of its ranks");
  KVIP_REQUIRE(a->rows >= 1 && a->shards >= 1 && a->shards <= 8, "topk_merge: 1..8 shards");
  cudaStream_t where = static_cast<cudaStream_t>(stream);
  const bool lists_aligned = a->peer_block || (((reinterpret_cast<uintptr_t>(a->cand_scores) | reinterpret_cast<uintptr_t>(a->cand_index)) & 7) == 0 &&
                                               a->shard_stride % 2 == 0 && a->row_stride % 2 == 0);
  if ((a->shards == 2 || a->shards == 4 || a->shards == 8) && lists_aligned) {
    // one CTA per shard on a cluster (needs `shards` free SMs of one GPC per row: rows beyond the first wave queue)
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(a->rows * a->shards, 1, 1);
    config.blockDim = dim3(kvip::kThreads, 1, 1);
    config.dynamicSmemBytes = sizeof(kvip::MergeHub);
    config.stream = where;
    if (uint32_t bad = kvip::raise_dynamic_smem(kvip::kSlotTopkMergeCluster, reinterpret_cast<const void*>(kvip::topk_merge_cluster),
                                                static_cast<int>(sizeof(kvip::MergeHub)), "topk_merge_cluster attribute"))
      return bad;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = a->shards;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (cudaLaunchKernelEx(&config, kvip::topk_merge_cluster, *a) != cudaSuccess) return kvip::check_launch("topk_merge_cluster");
    kvip::count_launch();
    return kvip::check_launch("topk_merge_cluster");
  }
  const size_t smem = (2u * a->shards + 1u) * KVIP_TOPK * sizeof(uint32_t);   // keys, indices, winners
  if (uint32_t bad = kvip::raise_dynamic_smem(kvip::kSlotTopkMerge, reinterpret_cast<const void*>(kvip::topk_merge),
                                              (2 * 8 + 1) * 2048 * 4, "topk_merge attribute"))
    return bad;
  kvip::topk_merge<<<a->rows, kvip::kThreads, smem, where>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("topk_merge");
}
