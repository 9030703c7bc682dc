// Byte movers and cache-state kernels: miss fetch from the host-mapped pool, dense gather of
// the selected KV rows, paged Index-cache ingest, SlotLRU commit and the ABC tail maps.
#include <cuda_fp8.h>
#include "common.cuh"

namespace kvip {
namespace {

// ---- fetch -------------------------------------------------------------------------------
// One warp per descriptor row, 16 bytes per lane per step: a 1152-byte row is 72 pieces, so a
// warp issues three fully coalesced 512-byte requests (the last one 128 bytes). The source is
// read through the device alias of pinned, mapped host memory; each request crosses the host
// link once and lands in the resident HBM slot.
// The descriptors of all requests form one flat list that the warps of a SMALL grid deal out round-robin: the
// host link, not the GPU, sets the pace (about 50 GB/s), 512 warps keep several hundred KB in flight, and a grid
// that leaves most SMs untouched lets the Index exchange (whose 1024-thread CTAs need an SM to themselves) and the
// gather of the hit entries run beside the fetch.
constexpr uint32_t kFetchThreads = 256;
constexpr uint32_t kFetchBlocks = 64;

__device__ __forceinline__ void copy_row_warp(uint8_t* dst, const uint8_t* src, uint32_t bytes, uint32_t lane) {
  const uint32_t pieces = bytes >> 4;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  uint4 v[3];
#pragma unroll
  for (uint32_t k = 0; k < 3; ++k)
    if (lane + 32u * k < pieces) v[k] = __ldcs(s + lane + 32u * k);
#pragma unroll
  for (uint32_t k = 0; k < 3; ++k)
    if (lane + 32u * k < pieces) d[lane + 32u * k] = v[k];
  for (uint32_t p = lane + 96u; p < pieces; p += 32u) d[p] = __ldcs(s + p);
}

__device__ __forceinline__ bool descriptor_ok(const KvipFetchArgs& a, int64_t source, int32_t dest, uint32_t slot) {
  return source >= 0 && static_cast<uint64_t>(source) + a.tokenBytes <= a.source_bytes && (source & 15) == 0 &&
         dest >= 0 && slot < a.outputStride;
}

// hot_valid = 1 for every accepted descriptor; the second half of a fetch that ran with defer_publication.
__global__ void __launch_bounds__(256) publish_residency(const KvipFetchArgs a) {
  const uint32_t b = blockIdx.y;
  if (a.row_status[b * 32u] != 0) return;
  // the descriptor lists hold kSlots entries per request: a count outside that range is not followed
  const uint32_t count = static_cast<uint32_t>(min(max(a.query_counts[b * 8u + 4], 0), static_cast<int32_t>(kSlots)));
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < count; i += gridDim.x * 256u) {
    const int64_t source = a.fetch_sources[static_cast<uint64_t>(b) * kSlots + i];
    const int32_t dest = a.fetch_destinations[static_cast<uint64_t>(b) * kSlots + i];
    const uint32_t slot = static_cast<uint32_t>(dest) - owner * a.outputStride;
    if (descriptor_ok(a, source, dest, slot) && slot < a.resident)
      a.hot_valid[static_cast<uint64_t>(owner) * a.resident + slot] = 1;
  }
}

__global__ void __launch_bounds__(kFetchThreads) fetch_rows(const KvipFetchArgs a) {
  // first descriptor of every request in the flat list (a failed request contributes none): all counts are loaded
  // at once, so the prologue costs one memory round trip whatever the batch
  __shared__ uint32_t first[1025];
  __shared__ uint32_t scan[33];
  const uint32_t tid = threadIdx.x, lane = tid & 31u;
  constexpr uint32_t kPer = 1024u / kFetchThreads;   // batch <= 1024
  uint32_t mine[kPer], sum = 0;
#pragma unroll
  for (uint32_t j = 0; j < kPer; ++j) {
    const uint32_t b = tid * kPer + j;
    mine[j] = b < a.batch && a.row_status[b * 32u] == 0
                  ? static_cast<uint32_t>(min(max(a.query_counts[b * 8u + 4], 0), static_cast<int32_t>(kSlots)))   // list capacity
                  : 0u;
    sum += mine[j];
  }
  uint32_t total;
  uint32_t before = block_exclusive_scan(sum, scan, &total);
#pragma unroll
  for (uint32_t j = 0; j < kPer; ++j) {
    first[tid * kPer + j] = before;
    before += mine[j];
  }
  if (tid == kFetchThreads - 1u) first[1024] = total;
  __syncthreads();
  const uint32_t warps = gridDim.x * (kFetchThreads / 32u);
  uint32_t b = 0;
  for (uint32_t item = blockIdx.x * (kFetchThreads / 32u) + (tid >> 5); item < total; item += warps) {
    while (first[b + 1] <= item) ++b;   // items ascend: the request index only moves forward (first[1024] = total ends it)
    const uint32_t i = item - first[b];
    const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
    const int64_t source = a.fetch_sources[static_cast<uint64_t>(b) * kSlots + i];
    const int32_t dest = a.fetch_destinations[static_cast<uint64_t>(b) * kSlots + i];
    const uint32_t slot = static_cast<uint32_t>(dest) - owner * a.outputStride;
    if (!descriptor_ok(a, source, dest, slot)) {
      // Record and skip the access (streaming.cpp:399-400 does the same range check). The Index row of the new
      // token already sits at this destination, so the slot must not keep the residency of the row it evicted:
      // it is revoked, and the request's update status gets the reference's code for a failed publication
      // (CompleteEarlyUpdate, index_cache_update.h:6-20).
      if (lane == 0) {
        atomicOr(a.row_status + b * 32u + 2, 1);
        if (a.status) atomicOr(a.status + b, 4);
        if (dest >= 0 && slot < a.resident) a.hot_valid[static_cast<uint64_t>(owner) * a.resident + slot] = 0;
      }
      continue;
    }
    copy_row_warp(a.pool + static_cast<uint64_t>(dest) * a.tokenBytes, a.source_base + source, a.tokenBytes, lane);
    if (lane == 0 && slot < a.resident && !a.defer_publication)
      a.hot_valid[static_cast<uint64_t>(owner) * a.resident + slot] = 1;
  }
}

// ---- dense gather --------------------------------------------------------------------------
// A warp gathers kGatherPerWarp consecutive entries of an output row: their slot numbers come with one load
// (one lane each), then every source row's three 512-byte requests are in flight together before the first
// store, so a warp keeps 4.5 KB moving instead of 1.1 KB behind a dependent index load.
constexpr uint32_t kGatherPerWarp = 4;

__global__ void __launch_bounds__(256) gather_rows(const KvipGatherArgs a) {
  const uint32_t row = blockIdx.y, lane = threadIdx.x & 31u;
  const uint32_t k0 = (blockIdx.x * 8u + (threadIdx.x >> 5)) * kGatherPerWarp;
  const uint32_t b = row / a.queries;
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  // two-phase gather: `wanted` has a bit per entry of this warp that belongs to the phase (hits first, beside the
  // fetch; the entries the fetch fills afterwards)
  uint32_t wanted = (1u << kGatherPerWarp) - 1u;
  if (a.miss_mask && a.phase) {
    const uint32_t missed = (a.miss_mask[static_cast<uint64_t>(row) * (kTop / 32u) + (k0 >> 5)] >> (k0 & 31u)) & wanted;
    wanted = a.phase == 2u ? missed : (~missed & wanted);
    if (!wanted) return;   // warp-uniform
  }
  const int32_t my_slot = lane < kGatherPerWarp ? a.slots[static_cast<uint64_t>(row) * kTop + k0 + lane] : -1;
  const uint32_t pieces = a.tokenBytes >> 4;
  uint8_t* dst0 = a.out + (static_cast<uint64_t>(row) * kTop + k0) * a.tokenBytes;
  if (pieces > 96u) {  // rows beyond 1536 bytes: one entry after the other
    for (uint32_t e = 0; e < kGatherPerWarp; ++e) {
      if (!((wanted >> e) & 1u)) continue;
      const int32_t slot = __shfl_sync(0xffffffffu, my_slot, e);
      uint4* d = reinterpret_cast<uint4*>(dst0 + static_cast<uint64_t>(e) * a.tokenBytes);
      if (slot < 0 || static_cast<uint32_t>(slot) >= a.outputStride) {
        for (uint32_t p = lane; p < pieces; p += 32u) d[p] = make_uint4(0, 0, 0, 0);
      } else {
        copy_row_warp(reinterpret_cast<uint8_t*>(d),
                      a.pool + (static_cast<uint64_t>(owner) * a.outputStride + static_cast<uint32_t>(slot)) * a.tokenBytes,
                      a.tokenBytes, lane);
      }
    }
    return;
  }
  uint4 v[kGatherPerWarp][3];
#pragma unroll
  for (uint32_t e = 0; e < kGatherPerWarp; ++e) {
    const int32_t slot = __shfl_sync(0xffffffffu, my_slot, e);
    const bool live = slot >= 0 && static_cast<uint32_t>(slot) < a.outputStride && ((wanted >> e) & 1u);
    const uint4* s = reinterpret_cast<const uint4*>(
        a.pool + (static_cast<uint64_t>(owner) * a.outputStride + (live ? static_cast<uint32_t>(slot) : 0u)) * a.tokenBytes);
#pragma unroll
    for (uint32_t k = 0; k < 3; ++k)
      v[e][k] = (live && lane + 32u * k < pieces) ? __ldcs(s + lane + 32u * k) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (uint32_t e = 0; e < kGatherPerWarp; ++e) {
    if (!((wanted >> e) & 1u)) continue;
    uint4* d = reinterpret_cast<uint4*>(dst0 + static_cast<uint64_t>(e) * a.tokenBytes);
#pragma unroll
    for (uint32_t k = 0; k < 3; ++k)
      if (lane + 32u * k < pieces) d[lane + 32u * k] = v[e][k];
  }
}

// ---- paged Index-cache ingest ----------------------------------------------------------------
__global__ void __launch_bounds__(128) ingest_rows(const KvipIngestArgs a) {
  const uint32_t row = blockIdx.x, d = threadIdx.x;
  const bool live = a.query_ends[row] > 0;
  int64_t source = 0;
  uint64_t target = row;  // padding rows land in owner 0 at distinct positions
  if (live) {
    source = a.slot_mapping[a.gather_indices[row]];
    target = static_cast<uint64_t>(a.row_owners[row / a.queries]) * a.history + static_cast<uint32_t>(a.query_ends[row] - 1);
  }
  if (!a.source_is_bf16) {
    a.keys[target * 128u + d] = reinterpret_cast<const uint8_t*>(a.source_keys)[static_cast<uint64_t>(source) * 128u + d];
    if (d == 0) a.scales[target] = a.source_scales[source];
    return;
  }
  // bf16 row -> FP8 e4m3 with one scale per token: scale = amax / 448 (1 for an all-zero row)
  __shared__ float warp_max[4];
  const float x = __uint_as_float(static_cast<uint32_t>(
                      reinterpret_cast<const uint16_t*>(a.source_keys)[static_cast<uint64_t>(source) * 128u + d]) << 16);
  float m = fabsf(x);
#pragma unroll
  for (uint32_t o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((d & 31u) == 0) warp_max[d >> 5] = m;
  __syncthreads();
  const float amax = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  a.keys[target * 128u + d] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x / scale, __NV_SATFINITE, __NV_E4M3));
  if (d == 0) a.scales[target] = scale;
}

// Import of whole spans of Index rows (prefill): a CTA takes 32 rows of one span, a warp 8 of them, a lane
// 4 bytes of the 128-byte key row.
__global__ void __launch_bounds__(128) ingest_span_rows(const KvipIngestSpanArgs a) {
  const int32_t* span = a.spans + static_cast<uint64_t>(blockIdx.y) * 8u;
  const int32_t owner = span[0], table_row = span[1], kind = span[2], first = span[3], tokens = span[4];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  if (static_cast<uint32_t>(owner) >= a.owners || first < 0 || tokens <= 0) return;
#pragma unroll
  for (uint32_t j = 0; j < 8u; ++j) {
    const uint32_t i = blockIdx.x * 32u + warp * 8u + j;
    if (i >= static_cast<uint32_t>(tokens)) break;
    int64_t source, position;
    if (kind == 0) {
      position = static_cast<int64_t>(first) + i;
      const uint64_t page = static_cast<uint64_t>(position) / a.block;
      const bool ok = static_cast<uint32_t>(table_row) < a.table_rows && page < a.table_stride;
      source = ok ? static_cast<int64_t>(a.block_table[static_cast<uint64_t>(table_row) * a.table_stride + page]) * a.block +
                        static_cast<int64_t>(static_cast<uint64_t>(position) % a.block)
                  : -1;
    } else {
      const uint64_t token = static_cast<uint64_t>(first) + i;
      const bool ok = token < a.batch_tokens;
      source = ok ? a.slot_mapping[token] : -1;
      position = ok ? a.positions[token] : -1;
    }
    if (source < 0 || static_cast<uint64_t>(source) >= a.source_rows || position < 0 ||
        position >= static_cast<int64_t>(a.history)) {
      if (lane == 0 && a.errors) atomicAdd(a.errors, 1);
      continue;
    }
    const uint64_t target = static_cast<uint64_t>(owner) * a.history + static_cast<uint64_t>(position);
    reinterpret_cast<uint32_t*>(a.keys + target * 128u)[lane] =
        reinterpret_cast<const uint32_t*>(a.source_keys + static_cast<uint64_t>(source) * 128u)[lane];
    if (lane == 0) a.scales[target] = a.source_scales[source];
  }
}

// ---- SlotLRU commit ---------------------------------------------------------------------------
// One CTA per row. The set of touched slots lives in shared memory (a 16 KiB bitmap covers the 131072
// slots a resident pool can have); the list is compacted in place in chunks of 32768 entries, every
// thread holding 32 consecutive entries in registers, so a 25 % pool of a 128k context is one chunk:
// one round of loads, one block scan, one round of stores.
constexpr uint32_t kLruThreads = 1024;
constexpr uint32_t kLruPer = 32;
constexpr uint32_t kLruMaxWords = 4096;

__global__ void __launch_bounds__(kLruThreads) lru_commit(const KvipLruArgs a) {
  __shared__ uint32_t touched_bits[kLruMaxWords];
  __shared__ uint32_t scan[33];
  __shared__ uint32_t unique_count;
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  const uint32_t active = min(static_cast<uint32_t>(max(a.active[row], 0)), a.capacity);
  const uint32_t active_words = (active + 31u) >> 5;
  int32_t* order = a.order + static_cast<uint64_t>(row) * a.capacity;
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(a.bitmap) + static_cast<uint64_t>(row) * a.words;
  int32_t* slots = a.slots + static_cast<uint64_t>(row) * kLruSlots;
  int32_t* reserved = a.reserved_hot ? a.reserved_hot + static_cast<uint64_t>(row) * a.resident : nullptr;
  const int32_t* touched = a.touched + static_cast<uint64_t>(row) * a.touched_stride;

  if (tid == 0) unique_count = 0;
  for (uint32_t w = tid; w < active_words; w += kLruThreads) touched_bits[w] = 0;
  for (uint32_t w = tid; w < a.words; w += kLruThreads) bitmap[w] = 0;
  if (reserved)
    for (uint32_t i = tid; i < kLruSlots; i += kLruThreads) {
      const int32_t old = slots[i];
      if (old >= 0 && static_cast<uint32_t>(old) < a.resident) reserved[old] = -1;
    }
  __syncthreads();
  // 1. distinct touched slots -> bitmap
  uint32_t mine = 0;
  for (uint32_t i = tid; i < a.touched_stride; i += kLruThreads) {
    const int32_t s = touched[i];
    if (s < 0 || static_cast<uint32_t>(s) >= active) continue;
    const uint32_t bit = 1u << (s & 31);
    if (!(atomicOr(touched_bits + (s >> 5), bit) & bit)) ++mine;
  }
  if (mine) atomicAdd(&unique_count, mine);
  __syncthreads();
  const uint32_t unique = unique_count;
  if (unique) {
    // 2. drop the touched slots from the list, keeping the order of the rest. In place: a chunk is fully
    //    in registers before anything is written, and writes never pass the reads. Every warp owns a
    //    contiguous run of the chunk (32 groups of 32 entries), so loads and stores are coalesced and the
    //    ranks inside a group come from a ballot; one block scan per chunk orders the warps.
    uint32_t kept_total = 0;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    for (uint32_t start = 0; start < active; start += kLruThreads * kLruPer) {
      int32_t v[kLruPer];
      uint32_t keep_mask[kLruPer];
      const uint32_t warp_base = start + warp * (32u * kLruPer);
      uint32_t warp_kept = 0;
#pragma unroll
      for (uint32_t j = 0; j < kLruPer; ++j) {
        const uint32_t p = warp_base + j * 32u + lane;
        v[j] = p < active ? order[p] : -1;
      }
#pragma unroll
      for (uint32_t j = 0; j < kLruPer; ++j) {
        const bool keep = v[j] >= 0 && !((touched_bits[v[j] >> 5] >> (v[j] & 31)) & 1u);
        keep_mask[j] = __ballot_sync(0xffffffffu, keep);
        warp_kept += __popc(keep_mask[j]);
      }
      uint32_t total;
      // one value per warp: lane 0 carries the warp's count into the block scan
      uint32_t offset = kept_total + block_exclusive_scan(lane == 0 ? warp_kept : 0u, scan, &total);
      offset = __shfl_sync(0xffffffffu, offset, 0);
#pragma unroll
      for (uint32_t j = 0; j < kLruPer; ++j) {
        if ((keep_mask[j] >> lane) & 1u) order[offset + __popc(keep_mask[j] & ((1u << lane) - 1u))] = v[j];
        offset += __popc(keep_mask[j]);
      }
      kept_total += total;
      __syncthreads();
    }
    // 3. append the touched slots in ascending slot number
    const uint32_t per = (active_words + kLruThreads - 1u) / kLruThreads;
    uint32_t local = 0;
    for (uint32_t w = tid * per; w < (tid + 1u) * per && w < active_words; ++w) local += __popc(touched_bits[w]);
    uint32_t out = kept_total + block_exclusive_scan(local, scan, nullptr);
    for (uint32_t w = tid * per; w < (tid + 1u) * per && w < active_words; ++w) {
      uint32_t bits = touched_bits[w];
      while (bits) {
        order[out++] = static_cast<int32_t>(w * 32u + __ffs(bits) - 1u);
        bits &= bits - 1u;
      }
    }
    __syncthreads();
  }
  // 4. victims = the oldest min(2048, active) slots, their bitmap and inverse map
  for (uint32_t i = tid; i < kLruSlots; i += kLruThreads) {
    const int32_t s = i < active ? order[i] : -1;
    slots[i] = s;
    if (s >= 0) {
      atomicOr(bitmap + (s >> 5), 1u << (s & 31));
      if (reserved && static_cast<uint32_t>(s) < a.resident) reserved[s] = static_cast<int32_t>(i);
    }
  }
  if (tid == 0) a.unique[row] = static_cast<int32_t>(unique);
}

// ---- ABC tail maps -------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) abc_rows(int32_t* t2s, int32_t* s2t, const int32_t* descriptors,
                                               uint32_t rows_per_group, uint32_t pool, uint32_t tokens,
                                               uint32_t slots, uint32_t history, uint32_t tail) {
  const int32_t* d = descriptors + (static_cast<uint64_t>(blockIdx.x) * rows_per_group + blockIdx.y) * 4u;
  const int32_t layer = d[0], owner = d[1], begin = d[2], end = d[3];
  int32_t* forward = t2s + (static_cast<uint64_t>(layer) * pool + owner) * tokens;
  int32_t* reverse = s2t + (static_cast<uint64_t>(layer) * pool + owner) * slots + history;
  for (int32_t t = begin + static_cast<int32_t>(threadIdx.x); t < end; t += 256)
    forward[t] = static_cast<int32_t>(history) + t % static_cast<int32_t>(tail);
  // reverse[j] = the last token of [begin, end) that maps to ring slot j, or -1
  for (uint32_t j = threadIdx.x; j < tail; j += 256) {
    int32_t value = -1;
    if (end > begin) {
      const int32_t last = end - 1;
      const int32_t back = ((last - static_cast<int32_t>(j)) % static_cast<int32_t>(tail) + static_cast<int32_t>(tail)) %
                           static_cast<int32_t>(tail);
      const int32_t t = last - back;
      if (t >= begin) value = t;
    }
    reverse[j] = value;
  }
}

// ---- appended host pages ---------------------------------------------------------------------------
// One CTA per appended page; the lanes cover the page's tokens.
__global__ void __launch_bounds__(128) publish_pages(const KvipPagesArgs a) {
  const int64_t* row = a.rows + static_cast<uint64_t>(blockIdx.x) * 3u;
  const int64_t index = row[0], address = row[1], clear = row[2];
  const uint64_t per_owner = static_cast<uint64_t>(a.groups) * a.pages;
  const bool bad = index < 0 || static_cast<uint64_t>(index) >= per_owner * a.owners ||
                   (clear >= 0 && static_cast<uint64_t>(clear) + a.block > a.map_entries);
  if (bad) {
    if (threadIdx.x == 0 && a.errors) atomicAdd(a.errors, 1);
    return;
  }
  if (threadIdx.x == 0) {
    a.addresses[index] = address;
    a.valid[index] = 1;
  }
  if (clear >= 0)
    for (uint32_t lane = threadIdx.x; lane < a.block; lane += blockDim.x) a.token_to_slot[clear + lane] = -1;
  if (a.fused_table) {
    const uint64_t owner = static_cast<uint64_t>(index) / per_owner;
    const uint32_t group = static_cast<uint32_t>(static_cast<uint64_t>(index) / a.pages % a.groups);
    const uint64_t page = static_cast<uint64_t>(index) % a.pages;
    int64_t* table = reinterpret_cast<int64_t*>(a.fused_table[group * 2u]);
    const int64_t bytes = a.fused_table[group * 2u + 1u];
    if (table)
      for (uint32_t lane = threadIdx.x; lane < a.block; lane += blockDim.x) {
        const uint64_t token = page * a.block + lane;
        if (token < a.history) table[owner * a.history + token] = address + static_cast<int64_t>(lane) * bytes;
      }
  }
}

}  // namespace

uint32_t launch_fetch(const KvipFetchArgs& a, cudaStream_t stream) {
  fetch_rows<<<kFetchBlocks, kFetchThreads, 0, stream>>>(a);
  count_launch();
  return check_launch("fetch_rows");
}

uint32_t launch_publish_residency(const KvipFetchArgs& a, cudaStream_t stream) {
  dim3 grid(4, a.batch);
  publish_residency<<<grid, 256, 0, stream>>>(a);
  count_launch();
  return check_launch("publish_residency");
}

uint32_t launch_gather(const KvipGatherArgs& a, cudaStream_t stream) {
  dim3 grid(kTop / (8u * kGatherPerWarp), a.rows);
  gather_rows<<<grid, 256, 0, stream>>>(a);
  count_launch();
  return check_launch("gather_rows");
}

}  // namespace kvip

extern "C" uint32_t kvip_b200_fetch(const KvipFetchArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->source_base && a->fetch_sources && a->fetch_destinations && a->query_counts &&
                   a->row_status && a->pool && a->hot_valid, "fetch: null pointer");
  KVIP_REQUIRE(a->tokenBytes >= 16 && a->tokenBytes % 16 == 0, "fetch: token bytes must be a multiple of 16");
  KVIP_REQUIRE((reinterpret_cast<uintptr_t>(a->pool) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a->source_base) & 15u) == 0,
               "fetch: pool and source base must be 16-byte aligned");
  KVIP_REQUIRE(a->batch >= 1 && a->batch <= 1024 && a->outputStride >= a->resident, "fetch: geometry (batch 1..1024)");
  return kvip::launch_fetch(*a, static_cast<cudaStream_t>(stream));
}

extern "C" uint32_t kvip_b200_publish_residency(const KvipFetchArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->fetch_sources && a->fetch_destinations && a->query_counts && a->row_status && a->hot_valid,
               "publish_residency: null pointer");
  KVIP_REQUIRE(a->batch >= 1 && a->outputStride >= a->resident, "publish_residency: geometry");
  return kvip::launch_publish_residency(*a, static_cast<cudaStream_t>(stream));
}

extern "C" uint32_t kvip_b200_gather(const KvipGatherArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->pool && a->slots && a->out, "gather: null pointer");
  KVIP_REQUIRE(a->tokenBytes >= 16 && a->tokenBytes % 16 == 0, "gather: token bytes must be a multiple of 16");
  KVIP_REQUIRE((reinterpret_cast<uintptr_t>(a->pool) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a->out) & 15u) == 0,
               "gather: pool and output must be 16-byte aligned");
  KVIP_REQUIRE(a->rows >= 1 && a->queries >= 1 && a->rows % a->queries == 0, "gather: rows must be batch*queries");
  KVIP_REQUIRE(a->phase <= 2u && (a->phase == 0u || a->miss_mask), "gather: phases 1 and 2 need the miss mask");
  return kvip::launch_gather(*a, static_cast<cudaStream_t>(stream));
}

namespace kvip {
namespace {
// QueryInputs.pack / bind_positions as one gather kernel: row r of the bound buffers takes token
// gather_indices[r] of the caller's tensors (adapters/vllm/inputs.py:121-152 does this with index_select calls).
__global__ void __launch_bounds__(256) pack_rows(const KvipPackArgs a) {
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  int64_t token = a.gather_indices[row];
  if (token < 0 || token >= static_cast<int64_t>(a.tokens)) token = 0;
  if (a.query_src) {
    const uint4* src = reinterpret_cast<const uint4*>(a.query_src + static_cast<uint64_t>(token) * a.query_row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(a.query_dst + static_cast<uint64_t>(row) * a.query_row_bytes);
    for (uint32_t i = tid; i < a.query_row_bytes / 16u; i += 256u) dst[i] = src[i];
  }
  if (a.weights_src) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.weights_src + static_cast<uint64_t>(token) * a.weights_row_bytes);
    uint32_t* dst = reinterpret_cast<uint32_t*>(a.weights_dst + static_cast<uint64_t>(row) * a.weights_row_bytes);
    for (uint32_t i = tid; i < a.weights_row_bytes / 4u; i += 256u) dst[i] = src[i];
  }
  if (a.scale_src)
    for (uint32_t i = tid; i < a.heads; i += 256u)
      a.scale_dst[static_cast<uint64_t>(row) * a.heads + i] = a.scale_src[static_cast<uint64_t>(token) * a.heads + i];
  if (a.positions_src && tid == 0) {
    const int64_t end = (a.positions_src[token] + 1) * a.query_valid[row];
    a.position_scratch[row] = end;
    a.query_ends[row] = static_cast<int32_t>(end);
  }
}
}  // namespace
}  // namespace kvip

extern "C" uint32_t kvip_b200_pack_inputs(const KvipPackArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->gather_indices && a->rows >= 1 && a->tokens >= 1, "pack_inputs: null pointer or empty batch");
  KVIP_REQUIRE(!a->query_src || (a->query_dst && a->query_row_bytes % 16u == 0 &&
                                 (reinterpret_cast<uintptr_t>(a->query_src) & 15u) == 0 &&
                                 (reinterpret_cast<uintptr_t>(a->query_dst) & 15u) == 0),
               "pack_inputs: query rows must be 16-byte aligned multiples of 16 bytes");
  KVIP_REQUIRE(!a->weights_src || (a->weights_dst && a->weights_row_bytes % 4u == 0 &&
                                   (reinterpret_cast<uintptr_t>(a->weights_src) & 3u) == 0),
               "pack_inputs: weight rows must be multiples of 4 bytes");
  KVIP_REQUIRE(!a->scale_src || a->scale_dst, "pack_inputs: scale destination missing");
  KVIP_REQUIRE(!a->positions_src || (a->query_valid && a->position_scratch && a->query_ends),
               "pack_inputs: position outputs missing");
  kvip::pack_rows<<<a->rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("pack_rows");
}

extern "C" uint32_t kvip_b200_ingest(const KvipIngestArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->source_keys && a->slot_mapping && a->gather_indices && a->query_ends && a->row_owners &&
                   a->keys && a->scales, "ingest: null pointer");
  KVIP_REQUIRE(a->source_is_bf16 || a->source_scales, "ingest: FP8 sources need their scales");
  KVIP_REQUIRE(a->batch >= 1 && a->queries >= 1 && a->queries <= KVIP_MAX_QUERIES, "ingest: bad batch/queries");
  kvip::ingest_rows<<<a->batch * a->queries, 128, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("ingest_rows");
}

extern "C" uint32_t kvip_b200_ingest_spans(const KvipIngestSpanArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->source_keys && a->source_scales && a->block_table && a->slot_mapping && a->positions && a->spans &&
                   a->keys && a->scales, "ingest_spans: null pointer");
  KVIP_REQUIRE(a->owners >= 1 && a->history >= 1 && a->block >= 1 && a->table_stride >= 1, "ingest_spans: geometry");
  KVIP_REQUIRE((reinterpret_cast<uintptr_t>(a->source_keys) & 3u) == 0 && (reinterpret_cast<uintptr_t>(a->keys) & 3u) == 0,
               "ingest_spans: key rows must be 4-byte aligned");
  if (a->count == 0 || a->max_tokens == 0) return 0u;
  KVIP_REQUIRE(a->count <= 65535u, "ingest_spans: at most 65535 spans per launch");
  dim3 grid((a->max_tokens + 31u) / 32u, a->count);
  kvip::ingest_span_rows<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("ingest_span_rows");
}

extern "C" uint32_t kvip_b200_lru_commit(const KvipLruArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->order && a->slots && a->bitmap && a->unique && a->touched && a->active, "lru_commit: null pointer");
  KVIP_REQUIRE(a->rows >= 1 && a->capacity >= 1 && a->words * 32u >= a->capacity, "lru_commit: bitmap too small");
  KVIP_REQUIRE(a->capacity <= kvip::kLruMaxWords * 32u, "lru_commit: at most 131072 slots per row");
  kvip::lru_commit<<<a->rows, kvip::kLruThreads, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("lru_commit");
}

extern "C" uint32_t kvip_b200_publish_pages(const KvipPagesArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->rows && a->addresses && a->valid && a->token_to_slot, "publish_pages: null pointer");
  KVIP_REQUIRE(a->owners >= 1 && a->groups >= 1 && a->pages >= 1 && a->block >= 1, "publish_pages: geometry");
  KVIP_REQUIRE(a->fused_table == nullptr || a->history >= 1, "publish_pages: fused groups need a history length");
  if (a->count == 0) return 0u;
  kvip::publish_pages<<<a->count, 128, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("publish_pages");
}

extern "C" uint32_t kvip_b200_update_abc(int32_t* token_to_slot, int32_t* slot_to_token, const int32_t* descriptors,
                                         uint32_t groups, uint32_t rows_per_group, uint32_t requests, uint32_t pool,
                                         uint32_t tokens, uint32_t slots, uint32_t history, uint32_t tail, void* stream) {
  KVIP_REQUIRE(token_to_slot && slot_to_token && descriptors, "update_abc: null pointer");
  KVIP_REQUIRE(groups >= 1 && requests >= 1 && requests <= rows_per_group && tail >= 1 && history + tail <= slots,
               "update_abc: geometry");
  dim3 grid(groups, requests);
  kvip::abc_rows<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(token_to_slot, slot_to_token, descriptors,
                                                                      rows_per_group, pool, tokens, slots, history, tail);
  kvip::count_launch();
  return kvip::check_launch("abc_rows");
}
