// LIDU: the serial-chain slot resolver behind kvip.lidu (out-parameter ABI).
//
// Restates A5LiduFusedBatchGetPrepareMtp (csrc/operators/lidu/op_kernel/
// a5_lidu_fused_batch_get_prepare_mtp.cpp: classify :195-221, dedup :223-263, clear :350-389,
// install :391-429, refill :431-458, descriptors :462-547, row checks :1290-1321, extra victims
// :1564-1741, outputs :2111-2196) as one CUDA kernel: one CTA per request; the CTA that finishes last
// compacts the per-request descriptors in request order.
// The reference numbers unique misses with an atomic counter, so which legal victim a miss gets
// is not fixed there; here unique misses are ordered by (query, TopK position) of their first
// occurrence, which makes every output a deterministic function of the inputs.
#include <cooperative_groups.h>
#include "common.cuh"

namespace cg = cooperative_groups;

namespace kvip {
namespace {

constexpr uint32_t kThreads = 1024;
constexpr uint32_t kBuckets = 16384;
constexpr uint32_t kEmpty = 0xffffffffu;
constexpr uint32_t kMaxCacheTokens = (1u << 17) + 20u * 128u;   // lidu_..._ops.cpp:17
constexpr uint32_t kRowWords = 3u * kSlots + 16u;               // scratch per request: three descriptor lists + control
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

// The two halves of a cluster barrier. A CTA may only touch another CTA's shared memory once that CTA is known to
// be running: every CTA arrives as its first action and waits just before its first remote store, so the
// barrier's latency hides behind the loads in between. (Both are no-ops in effect for a cluster of one CTA.)
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// One request: classification, miss numbering, victims, map update, destination rows. Leaves the request's
// unique miss tokens / slots and its control words in the scratch for the compaction.
//
// A request is served by a cluster of `ranks` CTAs. Only rank 0 resolves it; the others exist for ONE step,
// the gather of the 8192 token->slot entries of the request's TopK rows: one SM keeps only a few hundred
// loads in flight, so that gather alone took half of the kernel's time when one CTA did it. Every rank
// gathers its share and stores it into rank 0's shared memory; after one cluster barrier the helpers leave.
__device__ void lidu_request(const KvipLiduArgs& a, uint32_t* smem, cg::cluster_group& cluster, uint32_t ctas,
                             uint32_t cta) {
  const uint32_t r = blockIdx.x / ctas, tid = threadIdx.x, B = a.batch, T = a.packed_queries;
  int32_t* work = a.scratch + static_cast<uint64_t>(r) * kRowWords;
  int32_t* control = work + 3 * kSlots;  // 0 status, 1 unique, 2 new cursor (-1 = keep)
  __shared__ int32_t status;
  __shared__ uint32_t scan[33];
  cluster_arrive();   // "this CTA is resident": matched by the wait before the staged stores below, or by the
                      // wait of an early return (taken by every CTA of the cluster alike)
  if (tid == 0) status = 0;
  __syncthreads();
  // ---- layout of the packed query rows ---------------------------------------------------
  for (uint32_t i = tid; i < B; i += kThreads) {
    const int32_t lo = i ? a.actual_seq_lengths_query[i - 1] : 0, hi = a.actual_seq_lengths_query[i];
    if (hi - lo < 1 || hi - lo > 4 || hi > static_cast<int32_t>(T) || lo < 0) atomicMin(&status, kErrLayout);
  }
  __syncthreads();
  if (status) {  // the same on every rank: nobody reaches the second cluster barrier
    cluster_wait();
    if (cta != 0) return;
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
  if (!row_ok) {  // the same on every rank
    cluster_wait();
    if (cta != 0) return;
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
  uint32_t* ranks = keys + kBuckets;  // first occurrence of the bucket's token, later its unique-miss number
  int32_t* su_tokens = reinterpret_cast<int32_t*>(ranks + kBuckets);  // [8192] shared-memory copies of the
  int32_t* su_slots = su_tokens + kSlots;                             // [8192] unique-miss lists
  int32_t* t2s = a.token_to_slot_pool + static_cast<uint64_t>(pool) * a.source_capacity;
  int32_t* s2t = a.slot_to_token_pool + static_cast<uint64_t>(pool) * a.resident_capacity;
  // ---- gather of the map entries, spread over the cluster ---------------------------------------------
  // position p = 2048 * row + k of the request's TopK rows; CTA i of the cluster takes [i, i + 1) * 8192 / ctas. The staging
  // array is rank 0's su_tokens (not yet in use); invalid tokens and rows beyond q_count stage -1.
  {
    int32_t* staged = ctas > 1u ? cluster.map_shared_rank(su_tokens, 0) : su_tokens;
    const uint32_t per_thread = kSlots / (ctas * kThreads);  // 8, 4, 2 or 1
    const uint32_t first = cta * (kSlots / ctas) + tid;
    int32_t picked[8];
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
      const uint32_t p = first + i * kThreads;
      picked[i] = (i < per_thread && (p >> 11) < q_count) ? a.topk_indices[static_cast<uint64_t>(q_begin) * kTop + p] : -1;
    }
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
      const bool valid = picked[i] >= 0 && picked[i] < candidate;
      const int32_t mapped = t2s[valid ? picked[i] : 0];
      picked[i] = valid ? mapped : -1;
    }
    cluster_wait();   // every CTA of the cluster has started: rank 0's shared memory may be written
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i)
      if (i < per_thread) staged[first + i * kThreads] = picked[i];
  }
  if (cta == 0) {  // rank 0's own set-up overlaps the helpers' gathers
    for (uint32_t w = tid; w < a.bitmap_words; w += kThreads)
      prot[w] = static_cast<uint32_t>(a.miss_slot_bitmap[static_cast<uint64_t>(r) * a.bitmap_words + w]);
    for (uint32_t i = tid; i < kBuckets; i += kThreads) { keys[i] = kEmpty; ranks[i] = kEmpty; }
  }
  cluster.sync();  // every staged entry has landed in rank 0's shared memory (a block barrier for one CTA)
  if (cta != 0) return;
  // the first 2048 victims come from the caller's list: fetched now, needed after the classification
  const int32_t listed0 = a.miss_slots[static_cast<uint64_t>(r) * kLruSlots + tid];
  const int32_t listed1 = a.miss_slots[static_cast<uint64_t>(r) * kLruSlots + kThreads + tid];

  // ---- classify + miss-first compaction, all query rows at once ------------------------------------
  // A thread owns TopK positions 2*tid and 2*tid+1 of every query row; the per-row prefix sums of the four rows
  // travel through the block scan two rows per word (a row holds at most 2048 misses: 16 bits each).
  int32_t token[4][2], slot[4][2];
  uint32_t miss_flags = 0;  // bit 2q+j
  // (rows beyond q_count re-read the last row; they are masked afterwards)
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q) {
    const int2 pair = *reinterpret_cast<const int2*>(
        a.topk_indices + static_cast<uint64_t>(q_begin + min(q, q_count - 1u)) * kTop + tid * 2u);
    token[q][0] = pair.x;
    token[q][1] = pair.y;
  }
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q) {
    const int2 pair = *reinterpret_cast<const int2*>(su_tokens + q * kTop + tid * 2u);   // the staged map entries
    slot[q][0] = q < q_count ? pair.x : -1;
    slot[q][1] = q < q_count ? pair.y : -1;
  }
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q)
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      if (q < q_count) {
        if (token[q][j] < 0 || token[q][j] >= candidate) atomicMin(&status, kErrToken);
        const int32_t mapped = slot[q][j];
        if (!(mapped >= 0 && mapped < budget && !((prot[mapped >> 5] >> (mapped & 31)) & 1u))) {
          slot[q][j] = -1;
          miss_flags |= 1u << (2u * q + j);
        }
      }
    }
  auto pair_count = [](uint32_t flags, uint32_t q) { return static_cast<uint32_t>(__popc((flags >> (2u * q)) & 3u)); };
  uint32_t totals01, totals23;
  const uint32_t before01 = block_exclusive_scan(pair_count(miss_flags, 0) | (pair_count(miss_flags, 1) << 16), scan, &totals01);
  const uint32_t before23 = block_exclusive_scan(pair_count(miss_flags, 2) | (pair_count(miss_flags, 3) << 16), scan, &totals23);
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q) {
    if (q < q_count) {
    const uint32_t before = ((q < 2 ? before01 : before23) >> (16u * (q & 1u))) & 0xffffu;
    const uint32_t misses = ((q < 2 ? totals01 : totals23) >> (16u * (q & 1u))) & 0xffffu;
    int32_t* dest = a.destination_slots + static_cast<uint64_t>(q_begin + q) * kTop;
    // hits follow the misses, both in TopK order; the misses' slots are written after the install.
    // Hit slots are protected from the extra-victim scan.
    uint32_t hit_at = misses + (tid * 2u - before);
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j)
      if (!((miss_flags >> (2u * q + j)) & 1u)) {
        dest[hit_at++] = slot[q][j];
        atomicOr(prot + (slot[q][j] >> 5), 1u << (slot[q][j] & 31));
      }
    }
  }
  // hash insert of every miss; the first occurrence in (query row, TopK position) order keeps the bucket's rank
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q)
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      if (((miss_flags >> (2u * q + j)) & 1u) && token[q][j] >= 0 && token[q][j] < candidate) {
        const uint32_t i = q * kTop + tid * 2u + j;
        uint32_t h = hash14(static_cast<uint32_t>(token[q][j]));
        for (uint32_t probe = 0; probe < kBuckets; ++probe) {
          const uint32_t prev = atomicCAS(keys + h, kEmpty, static_cast<uint32_t>(token[q][j]));
          if (prev == kEmpty || prev == static_cast<uint32_t>(token[q][j])) {
            atomicMin(ranks + h, i);
            break;
          }
          h = (h + 1u) & (kBuckets - 1u);
        }
      }
    }
  __syncthreads();
  uint32_t fresh = 0;  // bit 2q+j: this position is the first occurrence of its token
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q)
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      if (((miss_flags >> (2u * q + j)) & 1u) && token[q][j] >= 0 && token[q][j] < candidate) {
        const uint32_t bucket = find_bucket(keys, static_cast<uint32_t>(token[q][j]));
        if (bucket != kEmpty && ranks[bucket] == q * kTop + tid * 2u + j) fresh |= 1u << (2u * q + j);
      }
    }
  uint32_t fresh01, fresh23;
  const uint32_t first01 = block_exclusive_scan(pair_count(fresh, 0) | (pair_count(fresh, 1) << 16), scan, &fresh01);
  const uint32_t first23 = block_exclusive_scan(pair_count(fresh, 2) | (pair_count(fresh, 3) << 16), scan, &fresh23);
  const uint32_t row_total[4] = {fresh01 & 0xffffu, fresh01 >> 16, fresh23 & 0xffffu, fresh23 >> 16};
  uint32_t unique = 0;
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q) {
    uint32_t offset = unique + (((q < 2 ? first01 : first23) >> (16u * (q & 1u))) & 0xffffu);
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j)
      if ((fresh >> (2u * q + j)) & 1u) {
        ranks[find_bucket(keys, static_cast<uint32_t>(token[q][j]))] = offset;  // every rank was compared before the scans
        su_tokens[offset++] = token[q][j];
      }
    unique += row_total[q];
  }
  __syncthreads();
  // ---- victims ---------------------------------------------------------------------------------
  int32_t new_cursor = -1;
  if (unique > kSlots) {
    if (tid == 0) atomicMin(&status, kErrCapacity);
  } else {
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {
      const uint32_t i = half * kThreads + tid;
      if (i < min(unique, kLruSlots)) {
        const int32_t s = half ? listed1 : listed0;
        if (s < 0 || s >= budget) atomicMin(&status, kErrResolved);
        su_slots[i] = s;
      }
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
            su_slots[kLruSlots + out] = static_cast<int32_t>(s);
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
  for (uint32_t base = 0; base < unique; base += 2u * kThreads) {  // two entries per thread: their loads overlap
    const uint32_t i0 = base + tid, i1 = base + kThreads + tid;
    const int32_t d0 = i0 < unique ? su_slots[i0] : 0, d1 = i1 < unique ? su_slots[i1] : 0;
    const int32_t v0 = s2t[d0], v1 = s2t[d1];
    const bool mapped0 = i0 < unique && v0 >= 0 && v0 < static_cast<int32_t>(a.source_capacity);
    const bool mapped1 = i1 < unique && v1 >= 0 && v1 < static_cast<int32_t>(a.source_capacity);
    const int32_t back0 = t2s[mapped0 ? v0 : 0], back1 = t2s[mapped1 ? v1 : 0];
    if (mapped0 && back0 == d0) t2s[v0] = -1;
    if (mapped1 && back1 == d1) t2s[v1] = -1;
  }
  __threadfence_block();
  __syncthreads();
  for (uint32_t i = tid; i < unique; i += kThreads) {
    t2s[su_tokens[i]] = su_slots[i];
    s2t[su_slots[i]] = su_tokens[i];
  }
  // every miss now lives in the slot of its token's unique-miss entry (the maps say the same after the install)
#pragma unroll
  for (uint32_t q = 0; q < 4; ++q) {
    if (q < q_count) {
      int32_t* dest = a.destination_slots + static_cast<uint64_t>(q_begin + q) * kTop;
      uint32_t miss_at = ((q < 2 ? before01 : before23) >> (16u * (q & 1u))) & 0xffffu;
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j)
        if ((miss_flags >> (2u * q + j)) & 1u)
          dest[miss_at++] = su_slots[ranks[find_bucket(keys, static_cast<uint32_t>(token[q][j]))]];
    }
  }
  // the unique misses' fetch descriptors, final values: into this request's scratch lists (the compaction then
  // only copies) or, when the call has one request, straight into the output lists
  {
    const bool single = B == 1u;
    int32_t* d_index = single ? a.indices : work;
    int32_t* d_offset = single ? a.offsets : work + kSlots;
    int32_t* d_out = single ? a.output_indices : work + 2 * kSlots;
    const int64_t table_row = static_cast<int64_t>((static_cast<int64_t>(pool) * a.num_layers + a.layer_id) * a.qcap);
    for (uint32_t base = 0; base < unique; base += 2u * kThreads) {  // two entries per thread: their loads overlap
      const uint32_t i0 = base + tid, i1 = base + kThreads + tid;
      const int32_t s0 = i0 < unique ? su_slots[i0] : 0, s1 = i1 < unique ? su_slots[i1] : 0;
      const int32_t b0 = a.resident_block_table[static_cast<uint64_t>(r) * a.resident_blocks + (s0 >> 7)];
      const int32_t b1 = a.resident_block_table[static_cast<uint64_t>(r) * a.resident_blocks + (s1 >> 7)];
      if (i0 < unique) {
        const int32_t t0 = su_tokens[i0];
        d_index[i0] = static_cast<int32_t>(table_row + (t0 >> 7));
        d_offset[i0] = (t0 & 127) * 656;
        d_out[i0] = b0 < 0 ? -1 : b0 * 128 + (s0 & 127);
      }
      if (i1 < unique) {
        const int32_t t1 = su_tokens[i1];
        d_index[i1] = static_cast<int32_t>(table_row + (t1 >> 7));
        d_offset[i1] = (t1 & 127) * 656;
        d_out[i1] = b1 < 0 ? -1 : b1 * 128 + (s1 & 127);
      }
    }
  }
  if (tid == 0) {
    control[0] = 0;
    control[1] = static_cast<int32_t>(unique);
    control[2] = new_cursor < 0 ? -1 : control[3];
  }
}

// Per-request results -> the packed descriptor lists, in request order; run by ONE CTA once every request is done.
__device__ void lidu_compact(const KvipLiduArgs& a) {
  __shared__ uint32_t offsets[1025];
  __shared__ uint32_t scan[33];
  const uint32_t tid = threadIdx.x, B = a.batch;
  uint32_t mine = 0;
  if (tid < B) {  // B <= 1024 = kThreads
    const int32_t* control = a.scratch + static_cast<uint64_t>(tid) * kRowWords + 3 * kSlots;
    const int32_t st = control[0], unique = control[1];
    if (st == 0) mine = static_cast<uint32_t>(unique);
    a.miss_counts[tid] = st == 0 ? unique : -1;
    const int32_t budget = a.cache_tokens[tid], cand = a.candidate_lens[tid], logical = a.logical_seq_lengths[tid];
    int32_t resident = 0;
    if (st == 0) {
      if (budget >= static_cast<int32_t>(kTop) && cand >= static_cast<int32_t>(kTop) && logical >= cand)
        resident = budget + logical - cand;
      else if (budget == 0 && logical >= 0)
        resident = logical;
    }
    a.resident_seq_lengths[tid] = resident;
    if (st == 0 && control[2] >= 0) a.eviction_cursors[a.req_pool_entries[tid]] = control[2];
  }
  uint32_t total;
  const uint32_t first = block_exclusive_scan(mine, scan, &total);
  if (tid < B) offsets[tid] = first;
  if (tid == 0) {
    offsets[B] = total;
    a.miss_counts[B] = static_cast<int32_t>(total);
  }
  __syncthreads();
  if (B == 1u) return;  // a single request wrote its descriptors in place
  // four descriptors per thread and round, all loads first: the request CTAs left final values in their scratch
  for (uint32_t base = 0; base < total; base += 4u * kThreads) {
    const int32_t* from[4];
    int32_t index[4], offset[4], output[4];
#pragma unroll
    for (uint32_t u = 0; u < 4; ++u) {
      const uint32_t o = base + u * kThreads + tid;
      uint32_t lo = 0, hi = B;  // the request r with offsets[r] <= o < offsets[r + 1]
      while (hi - lo > 1u) {
        const uint32_t mid = (lo + hi) >> 1;
        if (offsets[mid] <= o) lo = mid; else hi = mid;
      }
      from[u] = a.scratch + static_cast<uint64_t>(lo) * kRowWords + (o < total ? o - offsets[lo] : 0u);
    }
#pragma unroll
    for (uint32_t u = 0; u < 4; ++u) {
      index[u] = from[u][0];
      offset[u] = from[u][kSlots];
      output[u] = from[u][2 * kSlots];
    }
#pragma unroll
    for (uint32_t u = 0; u < 4; ++u) {
      const uint32_t o = base + u * kThreads + tid;
      if (o < total) {
        a.indices[o] = index[u];
        a.offsets[o] = offset[u];
        a.output_indices[o] = output[u];
      }
    }
  }
}

// One CTA per request; the CTA that finishes last (a ticket counter behind the per-request scratch, back at
// zero when the kernel ends) also compacts the descriptors. No CTA waits for another.
__device__ __forceinline__ int64_t device_time_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return static_cast<int64_t>(t);
}

__global__ void __launch_bounds__(kThreads, 1) lidu_requests(const KvipLiduArgs a) {
  extern __shared__ uint32_t smem[];
  __shared__ uint32_t last;
  // profiling[r, 0, 0..2] = device time (ns) when request r's CTA started, finished its request, and - for the
  // CTA that compacted - finished the kernel's work (0 otherwise); only when *profile_enabled is non-zero
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t ranks = cluster.num_blocks(), rank = cluster.block_rank();
  int64_t* stamps = rank == 0 && a.profiling && a.profile_enabled && *a.profile_enabled
                        ? a.profiling + static_cast<uint64_t>(blockIdx.x / ranks) * 256u : nullptr;
  if (stamps && threadIdx.x == 0) { stamps[0] = device_time_ns(); stamps[2] = 0; }
  lidu_request(a, smem, cluster, ranks, rank);
  if (rank != 0) return;   // helpers took part in the gather only
  if (stamps && threadIdx.x == 0) stamps[1] = device_time_ns();
  if (a.batch == 1u) {  // nobody else to wait for: the block barrier orders this CTA's own scratch writes
    __syncthreads();
    lidu_compact(a);
    __syncthreads();
    if (stamps && threadIdx.x == 0) stamps[2] = device_time_ns();
    return;
  }
  __threadfence();   // this request's scratch and control words are visible before the ticket is taken
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ticket = reinterpret_cast<uint32_t*>(a.scratch + static_cast<uint64_t>(a.batch) * kRowWords);
    const uint32_t taken = atomicAdd(ticket, 1u);
    last = taken == a.batch - 1u ? 1u : 0u;
    if (last) *ticket = 0u;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();   // acquire side: everything written before the other tickets were taken
  lidu_compact(a);
  __syncthreads();
  if (stamps && threadIdx.x == 0) stamps[2] = device_time_ns();
}

}  // namespace
}  // namespace kvip

extern "C" uint32_t kvip_b200_lidu_scratch_words(uint32_t batch) { return batch * kvip::kRowWords + 16u; }

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
  const size_t smem = (a->bitmap_words + 2u * kvip::kBuckets + 2u * kvip::kSlots) * sizeof(uint32_t);
  if (uint32_t bad = kvip::raise_dynamic_smem(kvip::kSlotLidu, reinterpret_cast<const void*>(kvip::lidu_requests),
                                              220 * 1024, "lidu attribute"))
    return bad;
  KVIP_REQUIRE(smem <= 220 * 1024, "lidu: bitmap does not fit in shared memory");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // helpers per request while the clusters still fit the GPU in one wave (a cluster of eight 1024-thread CTAs
  // needs eight free SMs of one GPC)
  const unsigned sms = kvip::device_sm_count();
  const unsigned ranks = 8u * a->batch <= (sms * 3u) / 4u ? 8u : (4u * a->batch <= (sms * 7u) / 8u ? 4u : (2u * a->batch <= sms ? 2u : 1u));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a->batch * ranks, 1, 1);
  config.blockDim = dim3(kvip::kThreads, 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = s;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = ranks;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, kvip::lidu_requests, *a) != cudaSuccess) return kvip::check_launch("lidu_requests");
  kvip::count_launch();
  return kvip::check_launch("lidu_requests");
}
