// LIDU: the serial-chain slot resolver behind kvip.lidu (out-parameter ABI).
//
// Restates A5LiduFusedBatchGetPrepareMtp (csrc/operators/lidu/op_kernel/
// a5_lidu_fused_batch_get_prepare_mtp.cpp: classify :195-221, dedup :223-263, clear :350-389,
// install :391-429, refill :431-458, descriptors :462-547, row checks :1290-1321, extra victims
// :1564-1741, outputs :2111-2196) as two CUDA kernels: one CTA per request, then one CTA that
// compacts the per-request descriptors in request order.
// The reference numbers unique misses with an atomic counter, so which legal victim a miss gets
// is not fixed there; here unique misses are ordered by (query, TopK position) of their first
// occurrence, which makes every output a deterministic function of the inputs.
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kThreads = 1024;
constexpr uint32_t kBuckets = 16384;
constexpr uint32_t kEmpty = 0xffffffffu;
constexpr uint32_t kRankTag = 0x80000000u;
constexpr uint32_t kMaxCacheTokens = (1u << 17) + 20u * 128u;   // lidu_..._ops.cpp:17
constexpr uint32_t kRowWords = 2u * kSlots + 16u;               // scratch per request
constexpr int32_t kErrLayout = -100, kErrRow = -101, kErrDuplicatePool = -102, kErrToken = -103,
                  kErrCapacity = -106, kErrNoSlots = -107, kErrResolved = -109;

__device__ __forceinline__ uint32_t hash14(uint32_t token) { return (token * 0x9e3779b9u) >> 18; }

__device__ __forceinline__ uint32_t find_bucket(const uint32_t* keys, uint32_t token) {
  uint32_t h = hash14(token);
  for (uint32_t probes = 0; probes < kBuckets; ++probes) {
    if (keys[h] == token) return h;
    h = (h + 1u) & (kBuckets - 1u);
  }
  return kEmpty;
}

__global__ void __launch_bounds__(kThreads) lidu_requests(const KvipLiduArgs a) {
  extern __shared__ uint32_t smem[];
  const uint32_t r = blockIdx.x, tid = threadIdx.x, B = a.batch, T = a.packed_queries;
  int32_t* work = a.scratch + static_cast<uint64_t>(r) * kRowWords;
  int32_t* u_tokens = work;            // [8192] unique miss tokens, first-occurrence order
  int32_t* u_slots = work + kSlots;    // [8192] their destination slots
  int32_t* control = work + 2 * kSlots;  // 0 status, 1 unique, 2 new cursor (-1 = keep)
  __shared__ int32_t status;
  __shared__ uint32_t scan[33];
  __shared__ uint32_t miss_total[4];
  if (tid == 0) status = 0;
  __syncthreads();
  // ---- layout of the packed query rows ---------------------------------------------------
  for (uint32_t i = tid; i < B; i += kThreads) {
    const int32_t lo = i ? a.actual_seq_lengths_query[i - 1] : 0, hi = a.actual_seq_lengths_query[i];
    if (hi - lo < 1 || hi - lo > 4 || hi > static_cast<int32_t>(T) || lo < 0) atomicMin(&status, kErrLayout);
  }
  __syncthreads();
  if (status) {
    for (uint32_t row = r; row < T; row += B)
      for (uint32_t k = tid; k < kTop; k += kThreads) a.destination_slots[static_cast<uint64_t>(row) * kTop + k] = -1;
    if (tid == 0) { control[0] = kErrLayout; control[1] = 0; control[2] = -1; }
    return;
  }
  const uint32_t q_begin = r ? static_cast<uint32_t>(a.actual_seq_lengths_query[r - 1]) : 0u;
  const uint32_t q_count = static_cast<uint32_t>(a.actual_seq_lengths_query[r]) - q_begin;
  const int32_t budget = a.cache_tokens[r], candidate = a.candidate_lens[r], pool = a.req_pool_entries[r];
  const bool row_ok = budget >= static_cast<int32_t>(kTop) && budget <= static_cast<int32_t>(kMaxCacheTokens) &&
                      budget <= static_cast<int32_t>(a.resident_capacity) && candidate >= static_cast<int32_t>(kTop) &&
                      candidate <= static_cast<int32_t>(a.source_capacity) &&
                      (static_cast<uint32_t>(candidate) + 127u) / 128u <= static_cast<uint64_t>(a.qcap) &&
                      (static_cast<uint32_t>(budget) + 127u) / 128u <= a.resident_blocks && pool >= 0 &&
                      pool < static_cast<int32_t>(a.pool_size) && pool < a.max_num_reqs;
  const bool padding = budget == 0 && candidate == 0 && a.logical_seq_lengths[r] == 1 && pool == a.max_num_reqs;
  if (!row_ok) {
    for (uint32_t q = 0; q < q_count; ++q)
      for (uint32_t k = tid; k < kTop; k += kThreads)
        a.destination_slots[static_cast<uint64_t>(q_begin + q) * kTop + k] = -1;
    if (tid == 0) { control[0] = padding ? 0 : kErrRow; control[1] = 0; control[2] = -1; }
    return;
  }
  for (uint32_t i = tid; i < B; i += kThreads)
    if (i != r && a.req_pool_entries[i] == pool && a.cache_tokens[i] >= static_cast<int32_t>(kTop))
      atomicMin(&status, kErrDuplicatePool);

  uint32_t* prot = smem;              // [bitmap_words] miss-slot membership, later + hit slots
  uint32_t* keys = prot + a.bitmap_words;
  uint32_t* ranks = keys + kBuckets;
  int32_t* t2s = a.token_to_slot_pool + static_cast<uint64_t>(pool) * a.source_capacity;
  int32_t* s2t = a.slot_to_token_pool + static_cast<uint64_t>(pool) * a.resident_capacity;
  for (uint32_t w = tid; w < a.bitmap_words; w += kThreads)
    prot[w] = static_cast<uint32_t>(a.miss_slot_bitmap[static_cast<uint64_t>(r) * a.bitmap_words + w]);
  for (uint32_t i = tid; i < kBuckets; i += kThreads) { keys[i] = kEmpty; ranks[i] = kEmpty; }
  if (tid < 4) miss_total[tid] = 0;
  __syncthreads();

  // ---- classify + miss-first compaction per query -----------------------------------------
  // class_slot (registers): 2 positions per thread per query
  uint32_t unique = 0;
  for (uint32_t q = 0; q < q_count; ++q) {
    const int32_t* topk = a.topk_indices + static_cast<uint64_t>(q_begin + q) * kTop;
    int32_t* dest = a.destination_slots + static_cast<uint64_t>(q_begin + q) * kTop;
    int32_t token[2], slot[2];
    uint32_t miss_flag = 0;
    for (uint32_t j = 0; j < 2; ++j) {
      const uint32_t k = tid * 2u + j;
      token[j] = topk[k];
      slot[j] = -1;
      if (token[j] >= 0 && token[j] < candidate) {
        const int32_t mapped = t2s[token[j]];
        if (mapped >= 0 && mapped < budget && !((prot[mapped >> 5] >> (mapped & 31)) & 1u)) slot[j] = mapped;
      } else {
        atomicMin(&status, kErrToken);
      }
      if (slot[j] < 0) miss_flag |= 1u << j;
    }
    uint32_t misses;
    const uint32_t before = block_exclusive_scan(__popc(miss_flag), scan, &misses);
    // hits follow the misses, both in TopK order
    uint32_t miss_at = before, hit_at = misses + (tid * 2u - before);
    for (uint32_t j = 0; j < 2; ++j) {
      if ((miss_flag >> j) & 1u) {
        dest[miss_at++] = -2 - static_cast<int32_t>(tid * 2u + j);  // resolved after the install
      } else {
        dest[hit_at++] = slot[j];
      }
    }
    if (tid == 0) miss_total[q] = misses;
    // hash insert of this query's misses, then rank first occurrences by position
    for (uint32_t j = 0; j < 2; ++j) {
      if (!((miss_flag >> j) & 1u) || token[j] < 0 || token[j] >= candidate) continue;
      const uint32_t i = q * kTop + tid * 2u + j;
      uint32_t h = hash14(static_cast<uint32_t>(token[j]));
      for (uint32_t probe = 0; probe < kBuckets; ++probe) {
        const uint32_t prev = atomicCAS(keys + h, kEmpty, static_cast<uint32_t>(token[j]));
        if (prev == kEmpty || prev == static_cast<uint32_t>(token[j])) {
          if (!(ranks[h] != kEmpty && (ranks[h] & kRankTag))) atomicMin(ranks + h, i);
          break;
        }
        h = (h + 1u) & (kBuckets - 1u);
      }
    }
    __syncthreads();
    uint32_t fresh = 0, bucket[2] = {0, 0};
    for (uint32_t j = 0; j < 2; ++j) {
      if (!((miss_flag >> j) & 1u) || token[j] < 0 || token[j] >= candidate) continue;
      bucket[j] = find_bucket(keys, static_cast<uint32_t>(token[j]));
      if (bucket[j] != kEmpty && ranks[bucket[j]] == q * kTop + tid * 2u + j) fresh |= 1u << j;
    }
    uint32_t added;
    uint32_t offset = unique + block_exclusive_scan(__popc(fresh), scan, &added);
    for (uint32_t j = 0; j < 2; ++j)
      if ((fresh >> j) & 1u) {
        ranks[bucket[j]] = kRankTag | offset;
        u_tokens[offset++] = token[j];
      }
    unique += added;
    __syncthreads();
  }
  // hit slots are protected from the extra-victim scan
  for (uint32_t q = 0; q < q_count; ++q) {
    const int32_t* dest = a.destination_slots + static_cast<uint64_t>(q_begin + q) * kTop;
    for (uint32_t k = miss_total[q] + tid; k < kTop; k += kThreads) {
      const int32_t s = dest[k];
      if (s >= 0) atomicOr(prot + (s >> 5), 1u << (s & 31));
    }
  }
  __syncthreads();
  // ---- victims ---------------------------------------------------------------------------------
  int32_t new_cursor = -1;
  if (unique > kSlots) {
    if (tid == 0) atomicMin(&status, kErrCapacity);
  } else {
    for (uint32_t i = tid; i < min(unique, kLruSlots); i += kThreads) {
      const int32_t s = a.miss_slots[static_cast<uint64_t>(r) * kLruSlots + i];
      if (s < 0 || s >= budget) atomicMin(&status, kErrResolved);
      u_slots[i] = s;
    }
    if (unique > kLruSlots) {
      const uint32_t extra = unique - kLruSlots;
      const uint32_t cursor = static_cast<uint32_t>(a.eviction_cursors[pool]) % static_cast<uint32_t>(budget);
      // ring order: [cursor, budget) then [0, cursor); ordered word list like hot_slot_selection.h
      const uint32_t first_words = (static_cast<uint32_t>(budget) - 1u) / 32u - cursor / 32u + 1u;
      const uint32_t second_words = cursor ? (cursor - 1u) / 32u + 1u : 0u;
      const uint32_t ordered = first_words + second_words;
      const uint32_t per = (ordered + kThreads - 1u) / kThreads;
      auto available = [&](uint32_t ordered_word, uint32_t* word_base) {
        uint32_t word, lo, hi;
        if (ordered_word < first_words) { word = cursor / 32u + ordered_word; lo = cursor; hi = static_cast<uint32_t>(budget); }
        else { word = ordered_word - first_words; lo = 0; hi = cursor; }
        const uint32_t base = word * 32u;
        uint32_t mask = 0xffffffffu;
        if (lo > base) mask &= 0xffffffffu << (lo - base);
        if (hi < base + 32u) mask &= hi > base ? (1u << (hi - base)) - 1u : 0u;
        *word_base = base;
        return ~prot[word] & mask;
      };
      uint32_t local = 0, base;
      for (uint32_t w = tid * per; w < (tid + 1u) * per && w < ordered; ++w) local += __popc(available(w, &base));
      uint32_t free_total;
      uint32_t out = block_exclusive_scan(local, scan, &free_total);
      if (free_total < extra) {
        if (tid == 0) atomicMin(&status, kErrNoSlots);
      } else {
        for (uint32_t w = tid * per; w < (tid + 1u) * per && w < ordered; ++w) {
          uint32_t bits = available(w, &base);
          while (bits && out < extra) {
            const uint32_t s = base + __ffs(bits) - 1u;
            u_slots[kLruSlots + out] = static_cast<int32_t>(s);
            if (out == extra - 1u) control[3] = static_cast<int32_t>((s + 1u) % static_cast<uint32_t>(budget));
            ++out;
            bits &= bits - 1u;
          }
        }
        new_cursor = 0;  // marker: control[3] holds the cursor
      }
    }
  }
  __syncthreads();
  if (status) {
    for (uint32_t q = 0; q < q_count; ++q)
      for (uint32_t k = tid; k < kTop; k += kThreads)
        a.destination_slots[static_cast<uint64_t>(q_begin + q) * kTop + k] = -1;
    if (tid == 0) { control[0] = status; control[1] = 0; control[2] = -1; }
    return;
  }
  // ---- clear, install, refill -----------------------------------------------------------------------
  for (uint32_t i = tid; i < unique; i += kThreads) {
    const int32_t d = u_slots[i];
    const int32_t v = s2t[d];
    if (v >= 0 && v < static_cast<int32_t>(a.source_capacity) && t2s[v] == d) t2s[v] = -1;
  }
  __threadfence_block();
  __syncthreads();
  for (uint32_t i = tid; i < unique; i += kThreads) {
    t2s[u_tokens[i]] = u_slots[i];
    s2t[u_slots[i]] = u_tokens[i];
  }
  __threadfence_block();
  __syncthreads();
  for (uint32_t q = 0; q < q_count; ++q) {
    const int32_t* topk = a.topk_indices + static_cast<uint64_t>(q_begin + q) * kTop;
    int32_t* dest = a.destination_slots + static_cast<uint64_t>(q_begin + q) * kTop;
    for (uint32_t k = tid; k < miss_total[q]; k += kThreads) {
      const int32_t position = -2 - dest[k];
      dest[k] = t2s[topk[position]];
    }
  }
  if (tid == 0) {
    control[0] = 0;
    control[1] = static_cast<int32_t>(unique);
    control[2] = new_cursor < 0 ? -1 : control[3];
  }
}

__global__ void __launch_bounds__(kThreads) lidu_compact(const KvipLiduArgs a) {
  __shared__ uint32_t offsets[1025];
  const uint32_t tid = threadIdx.x, B = a.batch;
  if (tid == 0) {
    uint32_t total = 0;
    for (uint32_t r = 0; r < B; ++r) {
      const int32_t* control = a.scratch + static_cast<uint64_t>(r) * kRowWords + 2 * kSlots;
      const int32_t st = control[0], unique = control[1];
      offsets[r] = total;
      if (st == 0) total += static_cast<uint32_t>(unique);
      a.miss_counts[r] = st == 0 ? unique : -1;
      const int32_t budget = a.cache_tokens[r], cand = a.candidate_lens[r], logical = a.logical_seq_lengths[r];
      int32_t resident = 0;
      if (st == 0) {
        if (budget >= static_cast<int32_t>(kTop) && cand >= static_cast<int32_t>(kTop) && logical >= cand)
          resident = budget + logical - cand;
        else if (budget == 0 && logical >= 0)
          resident = logical;
      }
      a.resident_seq_lengths[r] = resident;
      if (st == 0 && control[2] >= 0) a.eviction_cursors[a.req_pool_entries[r]] = control[2];
    }
    offsets[B] = total;
    a.miss_counts[B] = static_cast<int32_t>(total);
  }
  __syncthreads();
  for (uint32_t r = 0; r < B; ++r) {
    const int32_t* work = a.scratch + static_cast<uint64_t>(r) * kRowWords;
    const uint32_t count = offsets[r + 1] - offsets[r];
    const int64_t pool = a.req_pool_entries[r];
    for (uint32_t i = tid; i < count; i += kThreads) {
      const int32_t token = work[i], slot = work[kSlots + i];
      const uint32_t o = offsets[r] + i;
      a.indices[o] = static_cast<int32_t>((pool * a.num_layers + a.layer_id) * a.qcap + (token >> 7));
      a.offsets[o] = (token & 127) * 656;
      const int32_t block = a.resident_block_table[static_cast<uint64_t>(r) * a.resident_blocks + (slot >> 7)];
      a.output_indices[o] = block < 0 ? -1 : block * 128 + (slot & 127);
    }
  }
}

}  // namespace
}  // namespace kvip

extern "C" uint32_t kvip_b200_lidu_scratch_words(uint32_t batch) { return batch * kvip::kRowWords; }

extern "C" uint32_t kvip_b200_lidu(const KvipLiduArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->topk_indices && a->actual_seq_lengths_query && a->req_pool_entries && a->token_to_slot_pool &&
                   a->slot_to_token_pool && a->eviction_cursors && a->cache_tokens && a->candidate_lens &&
                   a->miss_slots && a->miss_slot_bitmap && a->resident_block_table && a->logical_seq_lengths &&
                   a->destination_slots && a->miss_counts && a->indices && a->offsets && a->output_indices &&
                   a->resident_seq_lengths && a->scratch, "lidu: null pointer");
  KVIP_REQUIRE(a->batch >= 1 && a->batch <= 1024, "lidu: batch must be in 1..1024");
  KVIP_REQUIRE(a->packed_queries >= a->batch && a->packed_queries <= 4 * a->batch, "lidu: 1..4 packed queries per request");
  KVIP_REQUIRE(a->resident_capacity >= KVIP_TOPK && a->source_capacity >= 1 &&
                   a->source_capacity <= (1u << 20) + 20u * 128u, "lidu: map capacities");
  KVIP_REQUIRE(a->bitmap_words * 32u >= (a->resident_capacity < kvip::kMaxCacheTokens ? a->resident_capacity : kvip::kMaxCacheTokens) ||
                   a->bitmap_words == 4176, "lidu: miss-slot bitmap too small");
  KVIP_REQUIRE(a->layer_id >= 0 && a->num_layers > 0 && a->layer_id < a->num_layers && a->max_num_reqs >= a->batch &&
                   a->qcap > 0, "lidu: access-table geometry");
  const size_t smem = (a->bitmap_words + 2u * kvip::kBuckets) * sizeof(uint32_t);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kvip::lidu_requests, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return kvip::check_launch("lidu attribute");
    configured = true;
  }
  KVIP_REQUIRE(smem <= 200 * 1024, "lidu: bitmap does not fit in shared memory");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  kvip::lidu_requests<<<a->batch, kvip::kThreads, smem, s>>>(*a);
  kvip::count_launch();
  if (uint32_t bad = kvip::check_launch("lidu_requests")) return bad;
  kvip::lidu_compact<<<1, kvip::kThreads, 0, s>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("lidu_compact");
}
