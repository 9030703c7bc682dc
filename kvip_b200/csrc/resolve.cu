// Classification of the selected positions, the resident-slot resolver and the service
// outputs: one CTA per request.
//
// Restates, for one CUDA block of 1024 threads, what the reference spreads over
// ClassifyTopkHalf/MergeClassifyBitmap (op_kernel/staged_topk_classify.h:9-46),
// StagedInitializeReady + StagedQuery (resolver_staged_dma2.h:83-237),
// PackStagedUrmaQuery/StoreFallbackSource (staged_urma_pack.h:6-71,
// common/lifetch/cache_metadata.h:32-44) and PublishQueryOutputs (streaming.cpp:66-90):
//
//   1. every selected position p of every query: hot  <=>  p < resident, hot_valid[owner,p],
//      reserved_hot[b,p] < 0 and p outside the ABC tail  ->  location p and protect bit p; a position
//      of the ABC tail that its ring of dedicated slots still holds  ->  resident + p % ring (known,
//      never protected, never a victim: cache_metadata.h:22-26, 100-105); otherwise a miss;
//   2. queries in order: misses are de-duplicated across queries with an open-addressing
//      hash (first occurrence wins by atomicMin on the TopK position), new misses are ranked
//      by ascending position with a block prefix sum, victims are the LRU candidates in list
//      order whose protect bit is clear, then - if those run out - the free slots of the
//      whole pool in ascending order; each assignment protects its slot;
//   3. per new slot: change record, exchange event, fetch source (address snapshot taken
//      before the Index rows move) and fetch destination;
//   4. logical_output / slot_output rows, routed through unpack_indices/output_valid when
//      bound.
//   5. one final-post record per (request, query): count, first descriptor, error
//      (PrepareFinalFetch, common/lifetch/final_post.h:5-12).
// Everything is ordered by prefix sums, so the slot map is a deterministic function of the
// inputs. The optional prefetch windows of this build stage rows in an area of their own and never
// write a victim slot, so the count of candidates already consumed by prefetch (`used`) is zero
// here: the reference's prefetch mapping has no counterpart, and every descriptor is non-conflicting.
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kThreads = 1024;
constexpr uint32_t kBuckets = 16384;  // >= 2 * 8192 distinct misses: probing always terminates
constexpr uint32_t kEmpty = 0xffffffffu;
constexpr uint32_t kRankTag = 0x80000000u;
constexpr uint32_t kMissing = 0xffffffffu;

__device__ __forceinline__ uint32_t sparse_hash(uint32_t token) {  // resolver.h:12
  return (token * 0x9e3779b9u) >> 18;                                 // 14 bits for 16384 buckets
}

__global__ void __launch_bounds__(kThreads) resolve_requests(const KvipResolveArgs a) {
  extern __shared__ uint32_t smem[];
  const uint32_t words = (a.resident + 31u) >> 5;
  uint32_t* bitmap = smem;                 // [words]
  uint32_t* keys = bitmap + words;         // [kBuckets]
  uint32_t* ranks = keys + kBuckets;       // [kBuckets]
  uint32_t* scan = ranks + kBuckets;       // [33]
  uint32_t* ctl = scan + 33;               // [8]: 0 = slots so far, 1 = error
  const uint32_t b = blockIdx.x, tid = threadIdx.x;
  const uint32_t Q = a.queries, R = a.resident, H = a.history;
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  const int32_t* selected = a.topk + static_cast<uint64_t>(b) * Q * kTop;
  uint32_t* loc = reinterpret_cast<uint32_t*>(a.locations) + static_cast<uint64_t>(b) * Q * kTop;
  const int32_t* valid = a.hot_valid + static_cast<uint64_t>(owner) * R;
  const int32_t* reserved = a.reserved_hot + static_cast<uint64_t>(b) * R;
  const int32_t* lru = a.lru_slots + static_cast<uint64_t>(b) * kLruSlots;
  int32_t* changes = a.changes + static_cast<uint64_t>(b) * kChangeCapacity;
  int32_t* change_slots = a.change_slots + static_cast<uint64_t>(b) * kChangeCapacity;
  int32_t* ev_src = a.events_src + static_cast<uint64_t>(b) * kSlots;
  int32_t* ev_dst = a.events_dst + static_cast<uint64_t>(b) * kSlots;
  int64_t* f_src = a.fetch_sources + static_cast<uint64_t>(b) * kSlots;
  int32_t* f_dst = a.fetch_destinations + static_cast<uint64_t>(b) * kSlots;
  const int64_t* address_row = a.addresses + static_cast<uint64_t>(owner) * a.address_stride;
  // ABC tail: positions [tail_begin, tail_end) live in the ring of outputStride - resident slots behind the hot ones
  const uint32_t ring = a.outputStride - R;
  uint32_t tail_begin = 0, tail_end = 0;
  if (a.tail_bounds && ring) {
    tail_begin = static_cast<uint32_t>(max(a.tail_bounds[b * 2u], 0));
    tail_end = static_cast<uint32_t>(max(a.tail_bounds[b * 2u + 1u], 0));
  }

  // ---- round init (v9_init_kernel, lifecycle.cpp:32-81): per-request scratch ----------
  for (uint32_t i = tid; i < words; i += kThreads) bitmap[i] = 0;
  for (uint32_t i = tid; i < kChangeCapacity; i += kThreads) {
    changes[i] = -1;
    change_slots[i] = i < kLruSlots ? lru[i] : -1;
  }
  if (tid < 8) ctl[tid] = 0;
  if (a.miss_mask)
    for (uint32_t i = tid; i < Q * (kTop / 32u); i += kThreads) a.miss_mask[static_cast<uint64_t>(b) * Q * (kTop / 32u) + i] = 0;
  __syncthreads();

  // ---- 1. classification of all queries ------------------------------------------------
  // A thread owns TopK positions 2*tid and 2*tid+1 of every query row and keeps their tokens and locations in
  // registers for the whole kernel. All token loads are issued first, then all residency lookups, so the four
  // rows cost one pair of memory round trips instead of one per row.
  int32_t token[KVIP_MAX_QUERIES][2];
  uint32_t where[KVIP_MAX_QUERIES][2];
#pragma unroll
  for (uint32_t q = 0; q < KVIP_MAX_QUERIES; ++q) {
    const int2 pair = *reinterpret_cast<const int2*>(selected + min(q, Q - 1u) * kTop + tid * 2u);
    token[q][0] = q < Q ? pair.x : -1;
    token[q][1] = q < Q ? pair.y : -1;
  }
  int32_t is_valid[KVIP_MAX_QUERIES][2], ordinal[KVIP_MAX_QUERIES][2];
#pragma unroll
  for (uint32_t q = 0; q < KVIP_MAX_QUERIES; ++q)
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      const bool resident_position = token[q][j] >= 0 && static_cast<uint32_t>(token[q][j]) < R;
      is_valid[q][j] = valid[resident_position ? token[q][j] : 0];
      ordinal[q][j] = reserved[resident_position ? token[q][j] : 0];
    }
#pragma unroll
  for (uint32_t q = 0; q < KVIP_MAX_QUERIES; ++q)
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      uint32_t slot = kMissing;
      if (q < Q && token[q][j] >= 0) {
        const uint32_t p = static_cast<uint32_t>(token[q][j]);
        if (p >= H) {
          atomicOr(ctl + 1, KVIP_ERR_TOKEN_RANGE);
        } else if (p >= tail_begin && p < tail_end) {
          if (p - tail_begin < ring) slot = R + p % ring;   // held by the ring; otherwise resolved like a cold position
        } else if (p < R && is_valid[q][j] != 0 && ordinal[q][j] < 0) {
          slot = static_cast<uint32_t>(token[q][j]);
          atomicOr(bitmap + (slot >> 5), 1u << (slot & 31u));
        }
      }
      where[q][j] = slot;
      if (q < Q) loc[q * kTop + tid * 2u + j] = slot;
    }
  if (a.miss_mask) {
    // bit k of a row: entry k is filled by this round's fetch. Entries 2*tid and 2*tid+1 are adjacent bits of one word.
#pragma unroll
    for (uint32_t q = 0; q < KVIP_MAX_QUERIES; ++q) {
      const uint32_t bits = (q < Q && token[q][0] >= 0 && where[q][0] == kMissing ? 1u : 0u) |
                            (q < Q && token[q][1] >= 0 && where[q][1] == kMissing ? 2u : 0u);
      if (bits) atomicOr(a.miss_mask + (static_cast<uint64_t>(b) * Q + q) * (kTop / 32u) + (tid >> 4), bits << ((tid & 15u) * 2u));
    }
  }
  // A request whose every selected position is resident (the steady state of a decode loop) needs neither the hash
  // table nor the per-query rounds below: nothing is unresolved. The vote is also the barrier after the classification.
  bool unresolved = false;
#pragma unroll
  for (uint32_t q = 0; q < KVIP_MAX_QUERIES; ++q)
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j)
      unresolved |= q < Q && token[q][j] >= 0 && where[q][j] == kMissing;
  const bool any_unresolved = __syncthreads_or(unresolved ? 1 : 0) != 0;   // positions beyond the history set ctl[1]
  if (any_unresolved) {
    for (uint32_t i = tid; i < kBuckets; i += kThreads) { keys[i] = kEmpty; ranks[i] = kEmpty; }
  } else if (tid < Q && !ctl[1]) {
    a.query_counts[b * 8u + tid] = 0;
  }
  __syncthreads();

  // ---- 2. queries in order ---------------------------------------------------------------
#pragma unroll
  for (uint32_t q = 0; q < KVIP_MAX_QUERIES; ++q) {
    if (q >= Q || ctl[1] || !any_unresolved) break;   // block-uniform
    const uint32_t begin = q * kTop, old_count = ctl[0];
    // 2a. hash insert, first occurrence by atomicMin on the position
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      const uint32_t i = begin + tid * 2u + j;
      if (token[q][j] < 0 || static_cast<uint32_t>(token[q][j]) >= H || where[q][j] != kMissing) continue;
      uint32_t h = sparse_hash(static_cast<uint32_t>(token[q][j])) & (kBuckets - 1u);
      for (uint32_t probe = 0; probe < kBuckets; ++probe) {
        const uint32_t prev = atomicCAS(keys + h, kEmpty, static_cast<uint32_t>(token[q][j]));
        if (prev == kEmpty || prev == static_cast<uint32_t>(token[q][j])) {
          // a tagged rank belongs to an earlier query: its slot is reused, not re-ranked
          if (!(ranks[h] != kEmpty && (ranks[h] & kRankTag))) atomicMin(ranks + h, i);
          break;
        }
        h = (h + 1u) & (kBuckets - 1u);
      }
    }
    __syncthreads();
    // 2b. rank the first occurrences by ascending position (2 consecutive positions / thread)
    uint32_t is_new[2] = {0, 0}, bucket[2] = {0, 0};
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      const uint32_t i = begin + tid * 2u + j;
      if (token[q][j] < 0 || static_cast<uint32_t>(token[q][j]) >= H || where[q][j] != kMissing) continue;
      uint32_t h = sparse_hash(static_cast<uint32_t>(token[q][j])) & (kBuckets - 1u), probes = 0;
      while (keys[h] != static_cast<uint32_t>(token[q][j]) && probes < kBuckets) { h = (h + 1u) & (kBuckets - 1u); ++probes; }
      if (probes == kBuckets) { atomicOr(ctl + 1, KVIP_ERR_HASH); continue; }
      bucket[j] = h;
      is_new[j] = ranks[h] == i ? 1u : 0u;
    }
    uint32_t added;
    uint32_t offset = block_exclusive_scan(is_new[0] + is_new[1], scan, &added);
    for (uint32_t j = 0; j < 2; ++j) {
      if (!is_new[j]) continue;
      const uint32_t rank = old_count + offset++;
      ranks[bucket[j]] = kRankTag | rank;
      ev_src[rank] = token[q][j];
    }
    __syncthreads();
    // 2c. victims from the LRU candidate list, in list order, unprotected only
    uint32_t allocated = 0;
    if (added) {
      uint32_t cand[2], free_flag[2];
      for (uint32_t j = 0; j < 2; ++j) {
        const int32_t slot = lru[tid * 2u + j];
        cand[j] = static_cast<uint32_t>(slot);
        if (slot < 0 || static_cast<uint32_t>(slot) >= R) {
          // entries of -1 pad a candidate list shorter than 2048; anything else is corrupt
          if (slot != -1) atomicOr(ctl + 1, KVIP_ERR_NO_SLOT);
          free_flag[j] = 0;
        } else {
          free_flag[j] = (bitmap[cand[j] >> 5] >> (cand[j] & 31u)) & 1u ? 0u : 1u;
        }
      }
      uint32_t available;
      uint32_t rank = block_exclusive_scan(free_flag[0] + free_flag[1], scan, &available);
      allocated = available < added ? available : added;
      for (uint32_t j = 0; j < 2; ++j) {
        if (!free_flag[j]) continue;
        if (rank < allocated) ev_dst[old_count + rank] = static_cast<int32_t>(cand[j]);
        ++rank;
      }
      __syncthreads();
      for (uint32_t i = tid; i < allocated; i += kThreads) {
        const uint32_t slot = static_cast<uint32_t>(ev_dst[old_count + i]);
        atomicOr(bitmap + (slot >> 5), 1u << (slot & 31u));
      }
      __syncthreads();
    }
    // 2d. fallback: free slots of the whole pool in ascending order (hot_slot_selection.h)
    if (allocated < added) {
      const uint32_t need = added - allocated;
      const uint32_t per = (words + kThreads - 1u) / kThreads;
      uint32_t local = 0;
      for (uint32_t w = tid * per; w < (tid + 1u) * per && w < words; ++w) {
        uint32_t mask = 0xffffffffu;
        if (w * 32u + 32u > R) mask = (1u << (R - w * 32u)) - 1u;
        local += __popc(~bitmap[w] & mask);
      }
      uint32_t free_total;
      uint32_t out = block_exclusive_scan(local, scan, &free_total);
      if (free_total < need) {
        if (tid == 0) atomicOr(ctl + 1, KVIP_ERR_NO_SLOT);
      } else {
        for (uint32_t w = tid * per; w < (tid + 1u) * per && w < words; ++w) {
          uint32_t mask = 0xffffffffu;
          if (w * 32u + 32u > R) mask = (1u << (R - w * 32u)) - 1u;
          uint32_t avail = ~bitmap[w] & mask;
          while (avail && out < need) {
            const uint32_t bit = __ffs(avail) - 1u;
            ev_dst[old_count + allocated + out] = static_cast<int32_t>(w * 32u + bit);
            ++out;
            avail &= avail - 1u;
          }
        }
      }
      __syncthreads();
      if (!ctl[1])
        for (uint32_t i = tid + allocated; i < added; i += kThreads) {
          const uint32_t slot = static_cast<uint32_t>(ev_dst[old_count + i]);
          atomicOr(bitmap + (slot >> 5), 1u << (slot & 31u));
        }
    }
    __syncthreads();
    if (ctl[1]) break;
    // 2e. publish locations of this query and the per-slot records
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      if (token[q][j] < 0 || where[q][j] != kMissing) continue;
      uint32_t h = sparse_hash(static_cast<uint32_t>(token[q][j])) & (kBuckets - 1u), probes = 0;
      while (keys[h] != static_cast<uint32_t>(token[q][j]) && probes < kBuckets) { h = (h + 1u) & (kBuckets - 1u); ++probes; }
      if (probes == kBuckets) { atomicOr(ctl + 1, KVIP_ERR_HASH); continue; }
      loc[begin + tid * 2u + j] = static_cast<uint32_t>(ev_dst[ranks[h] & ~kRankTag]);
    }
    for (uint32_t i = tid; i < added; i += kThreads) {
      const uint32_t rank = old_count + i;
      const int32_t token = ev_src[rank], slot = ev_dst[rank];
      const int32_t ordinal = reserved[slot];
      const uint32_t record = ordinal >= 0 ? static_cast<uint32_t>(ordinal) : kLruSlots + rank;
      change_slots[record] = slot;
      changes[record] = token;
      const int64_t source = address_row[token];
      // a source outside the pool fails the request HERE, before the Index rows move (streaming.cpp:399-400
      // range-checks the same descriptors): nothing is exchanged or fetched for it and it keeps no residency
      if (a.source_bytes && (source < 0 || (source & 15) != 0 ||
                             static_cast<uint64_t>(source) + a.tokenBytes > a.source_bytes))
        atomicOr(ctl + 1, KVIP_ERR_SOURCE);
      f_src[rank] = source;
      f_dst[rank] = static_cast<int32_t>(owner * a.outputStride) + slot;
    }
    __syncthreads();
    if (ctl[1]) break;   // a source address failed its range check
    if (tid == 0) {
      ctl[0] = old_count + added;
      a.query_counts[b * 8u + q] = static_cast<int32_t>(added);
    }
    __syncthreads();
  }
  __syncthreads();
  if (tid == 0) {
    const uint32_t error = ctl[1];
    for (uint32_t q = 0; q < 4; ++q)
      if (q >= Q || error) a.query_counts[b * 8u + q] = 0;
    a.query_counts[b * 8u + 4] = error ? 0 : static_cast<int32_t>(ctl[0]);
    a.change_count[b] = static_cast<int32_t>(kLruSlots + (error ? 0u : ctl[0]));
    a.row_status[b * 32u + 0] = static_cast<int32_t>(error);
    a.row_status[b * 32u + 1] = static_cast<int32_t>(ctl[0]);
  }
  __syncthreads();   // the final counts are in place
  if (a.final_posts && tid < 4u * 32u) {   // four 128-byte records, one word per thread
    const uint32_t q = tid >> 5, word = tid & 31u;
    const uint32_t error = ctl[1];
    uint32_t first = 0;
    for (uint32_t earlier = 0; earlier < q; ++earlier) first += static_cast<uint32_t>(a.query_counts[b * 8u + earlier]);
    const uint32_t count = static_cast<uint32_t>(a.query_counts[b * 8u + q]);
    const uint32_t value = word == 0u ? count : (word == 2u ? error : (word == 4u ? b * kSlots + first : (word == 5u ? count : 0u)));
    reinterpret_cast<uint32_t*>(a.final_posts + static_cast<uint64_t>(b) * 4u + q)[word] = value;
  }
}

// Service outputs: logical ids (before the Index rows move) and slots of every query row,
// routed to packed output rows (PrepareStagedQueryOutputs, staged_outputs.h:11-47).
__global__ void __launch_bounds__(256) publish_outputs(const KvipResolveArgs a) {
  const uint32_t out_row = blockIdx.x, Q = a.queries;
  const uint32_t k_begin = blockIdx.y * (kTop / 8u), k_end = k_begin + kTop / 8u;  // 8 CTAs per row
  int64_t src = out_row;
  bool live;
  if (a.unpack_indices && a.output_valid) {
    live = a.output_valid[out_row] != 0;
    src = live ? a.unpack_indices[out_row] : 0;
    if (src < 0 || src >= static_cast<int64_t>(a.batch) * Q) live = false;
  } else {
    live = !a.query_ends || a.query_ends[out_row] > 0;
  }
  int32_t* logical = a.logical_output + static_cast<uint64_t>(out_row) * kTop;
  int32_t* slots = a.slot_output + static_cast<uint64_t>(out_row) * kTop;
  const uint32_t b = static_cast<uint32_t>(src) / Q;
  if (live && a.row_status[b * 32u] != 0) live = false;
  if (!live) {
    for (uint32_t k = k_begin + threadIdx.x; k < k_end; k += 256) { logical[k] = -1; slots[k] = -1; }
    return;
  }
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  const int64_t* ids = a.logical_ids + static_cast<uint64_t>(owner) * a.history;
  const int32_t* selected = a.topk + static_cast<uint64_t>(src) * kTop;
  const int32_t* loc = a.locations + static_cast<uint64_t>(src) * kTop;
  for (uint32_t k = k_begin + threadIdx.x; k < k_end; k += 256) {
    const int32_t token = selected[k];
    logical[k] = token < 0 ? -1 : static_cast<int32_t>(ids[token]);
    slots[k] = loc[k];
  }
}

}  // namespace

uint32_t launch_resolve_requests(const KvipResolveArgs& a, cudaStream_t stream) {
  const uint32_t words = (a.resident + 31u) >> 5;
  const size_t smem = (words + 2u * kBuckets + 33u + 8u) * sizeof(uint32_t);
  if (uint32_t bad = raise_dynamic_smem(kSlotResolve, reinterpret_cast<const void*>(resolve_requests), 200 * 1024,
                                        "resolve attribute"))
    return bad;
  resolve_requests<<<a.batch, kThreads, smem, stream>>>(a);
  count_launch();
  return check_launch("resolve_requests");
}

uint32_t launch_publish_outputs(const KvipResolveArgs& a, cudaStream_t stream) {
  if (!a.logical_output || !a.slot_output) return 0;
  publish_outputs<<<dim3(a.batch * a.queries, 8), 256, 0, stream>>>(a);
  count_launch();
  return check_launch("publish_outputs");
}

uint32_t launch_resolve(const KvipResolveArgs& a, cudaStream_t stream) {
  if (uint32_t bad = launch_resolve_requests(a, stream)) return bad;
  return launch_publish_outputs(a, stream);
}

}  // namespace kvip

extern "C" uint32_t kvip_b200_resolve(const KvipResolveArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->topk && a->hot_valid && a->reserved_hot && a->lru_slots && a->logical_ids &&
                   a->addresses && a->locations && a->changes && a->change_slots && a->change_count &&
                   a->events_src && a->events_dst && a->query_counts && a->fetch_sources &&
                   a->fetch_destinations && a->row_status, "resolve: null pointer");
  KVIP_REQUIRE(a->tail_bounds == nullptr || (a->outputStride - a->resident >= 384 && (a->outputStride - a->resident) % 128 == 0),
               "resolve: ABC tail bounds need at least 384 dedicated slots behind the hot ones, in blocks of 128");
  KVIP_REQUIRE(a->batch >= 1 && a->queries >= 1 && a->queries <= KVIP_MAX_QUERIES, "resolve: bad batch/queries");
  KVIP_REQUIRE(a->resident >= KVIP_TOPK && a->resident <= 131072 && a->resident % 128 == 0,
               "resolve: resident must be in 2048..131072, multiple of 128");
  KVIP_REQUIRE(a->history >= a->resident && a->address_stride >= a->history, "resolve: history/address stride");
  KVIP_REQUIRE(a->outputStride >= a->resident, "resolve: output stride must cover the resident slots");
  return kvip::launch_resolve(*a, static_cast<cudaStream_t>(stream));
}
