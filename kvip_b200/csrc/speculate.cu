// Speculative prefetch windows: while the score kernel works on later key windows, rows of cold positions
// whose score already beats the resident threshold are copied from the host pool into a staging area in HBM;
// the final fetch then finds most of its missing rows there. Nothing here touches the slot maps, the LRU or
// the Index rows: speculation only changes where a missing row's bytes are read from.
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kStagedMax = 512;   // rows per request and round (prefetch_budget.h:7-17)

__device__ __forceinline__ void copy_row(uint8_t* dst, const uint8_t* src, uint32_t bytes, uint32_t lane) {
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

// ---- per-window bounds, and the round's counters back to zero ---------------------------------------
__global__ void __launch_bounds__(256) window_bounds(const KvipWindowArgs a) {
  const uint32_t rows = a.batch * a.queries;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < a.windows * rows; i += gridDim.x * blockDim.x) {
    const uint32_t w = i / rows, row = i % rows;
    const int32_t first = static_cast<int32_t>(a.first[w]), width = static_cast<int32_t>(a.first[w + 1]) - first;
    a.window_ends[i] = max(0, min(a.query_ends[row] - first, width));
    if (row < a.batch) a.window_lengths[w * a.batch + row] = max(0, min(a.key_lengths[row] - first, width));
    if (w == 0 && row < a.batch) {
      a.staged_count[row] = 0;
      a.staged_rows[row] = 0;
      if (a.staged_hits) a.staged_hits[row] = 0;
    }
  }
}

// ---- resident threshold: the smallest key of the prefix TopK -------------------------------------------
// Keys are the order-preserving unsigned image of the scores (sortable_key), as in the TopK itself.
__global__ void __launch_bounds__(256) resident_threshold(const KvipThresholdArgs a) {
  __shared__ uint32_t warp_min[8];
  __shared__ int warp_short[8];
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  uint32_t lowest = 0xffffffffu;
  int incomplete = 0;
  for (uint32_t k = tid; k < kTop; k += 256) {
    if (a.prefix_topk[static_cast<uint64_t>(row) * kTop + k] < 0) incomplete = 1;
    else lowest = min(lowest, sortable_key(a.prefix_scores[static_cast<uint64_t>(row) * kTop + k]));
  }
#pragma unroll
  for (uint32_t o = 16; o > 0; o >>= 1) {
    lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
    incomplete |= __shfl_xor_sync(0xffffffffu, incomplete, o);
  }
  if ((tid & 31u) == 0) { warp_min[tid >> 5] = lowest; warp_short[tid >> 5] = incomplete; }
  __syncthreads();
  if (tid == 0) {
    for (uint32_t w = 1; w < 8; ++w) { lowest = min(lowest, warp_min[w]); incomplete |= warp_short[w]; }
    // fewer than 2048 resident positions: threshold 0, every cold position may still be selected
    a.thresholds[row] = incomplete ? 0u : lowest;
  }
}

// ---- list the window's candidates ----------------------------------------------------------------
// One thread per cold position: it passes when any query row of the request scores it above that row's
// threshold. The request's list takes its source address while the round's limit lasts.
__global__ void __launch_bounds__(256) speculate_collect(const KvipSpeculateArgs a) {
  const uint32_t b = blockIdx.y;
  const uint32_t p = a.first + blockIdx.x * 256u + threadIdx.x;
  if (p >= a.last) return;
  const int32_t length = a.key_lengths[b];
  bool pass = false;
  for (uint32_t q = 0; q < a.queries; ++q) {
    const uint32_t row = b * a.queries + q;
    const int32_t bound = min(length, a.query_ends[row]);
    if (static_cast<int32_t>(p) < bound && sortable_key(a.scores[static_cast<uint64_t>(row) * a.scoreStride + p]) > a.thresholds[row])
      pass = true;
  }
  if (!pass) return;
  const uint32_t i = static_cast<uint32_t>(atomicAdd(a.staged_count + b, 1));
  if (i >= a.limit) return;   // over the limit: the count is clamped by the copy kernel
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  a.staged_sources[static_cast<uint64_t>(b) * a.capacity + i] = a.addresses[static_cast<uint64_t>(owner) * a.address_stride + p];
}

// ---- copy the listed rows into the staging area ------------------------------------------------------
// One CTA per request, one warp per row. A listed source that is out of range is replaced by -1 so that the
// final fetch never matches it.
__global__ void __launch_bounds__(512) speculate_copy(const KvipSpeculateArgs a) {
  const uint32_t b = blockIdx.x, lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t listed = min(static_cast<uint32_t>(a.staged_count[b]), a.limit);
  const uint32_t done = static_cast<uint32_t>(a.staged_rows[b]);
  for (uint32_t i = done + warp; i < listed; i += 16u) {
    int64_t* entry = a.staged_sources + static_cast<uint64_t>(b) * a.capacity + i;
    const int64_t source = *entry;
    const bool ok = source >= 0 && static_cast<uint64_t>(source) + a.tokenBytes <= a.source_bytes && (source & 15) == 0;
    __syncwarp();
    if (!ok) {
      if (lane == 0) *entry = -1;
      continue;
    }
    copy_row(a.staging + (static_cast<uint64_t>(b) * a.capacity + i) * a.tokenBytes, a.source_base + source, a.tokenBytes, lane);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    a.staged_count[b] = static_cast<int32_t>(listed);
    a.staged_rows[b] = static_cast<int32_t>(listed);
  }
}

// ---- the final fetch, with the staging area in front of the host pool ------------------------------------
constexpr uint32_t kFetchThreads = 256;
constexpr uint32_t kFetchBlocksPerRequest = 16;

struct StagedView {
  const int64_t* sources;
  const int32_t* rows;
  const uint8_t* staging;
  int32_t* hits;
  uint32_t capacity;
};

__global__ void __launch_bounds__(kFetchThreads) fetch_rows_staged(const KvipFetchArgs a, const StagedView view) {
  __shared__ int64_t staged[kStagedMax];
  const uint32_t b = blockIdx.y, lane = threadIdx.x & 31u;
  if (a.row_status[b * 32u] != 0) return;
  const uint32_t count = static_cast<uint32_t>(a.query_counts[b * 8u + 4]);
  if (blockIdx.x * (kFetchThreads / 32u) >= count) return;
  const uint32_t staged_rows = min(static_cast<uint32_t>(view.rows[b]), min(view.capacity, kStagedMax));
  for (uint32_t i = threadIdx.x; i < kStagedMax; i += kFetchThreads)
    staged[i] = i < staged_rows ? view.sources[static_cast<uint64_t>(b) * view.capacity + i] : -1;
  __syncthreads();
  const uint32_t owner = a.row_owners ? static_cast<uint32_t>(a.row_owners[b]) : b;
  const uint32_t warps = gridDim.x * (kFetchThreads / 32u);
  uint32_t served = 0;
  for (uint32_t i = blockIdx.x * (kFetchThreads / 32u) + (threadIdx.x >> 5); i < count; i += warps) {
    const int64_t source = a.fetch_sources[static_cast<uint64_t>(b) * kSlots + i];
    const int32_t dest = a.fetch_destinations[static_cast<uint64_t>(b) * kSlots + i];
    const uint32_t slot = static_cast<uint32_t>(dest) - owner * a.outputStride;
    const bool ok = source >= 0 && static_cast<uint64_t>(source) + a.tokenBytes <= a.source_bytes &&
                    (source & 15) == 0 && dest >= 0 && slot < a.outputStride;
    if (!ok) {  // as in fetch_rows: recorded, skipped, and the destination slot loses residency
      if (lane == 0) {
        atomicOr(a.row_status + b * 32u + 2, 1);
        if (a.status) atomicOr(a.status + b, 4);
        if (dest >= 0 && slot < a.resident) a.hot_valid[static_cast<uint64_t>(owner) * a.resident + slot] = 0;
      }
      continue;
    }
    uint32_t found = 0xffffffffu;
    for (uint32_t base = 0; base < staged_rows; base += 32u) {
      const uint32_t match = __ballot_sync(0xffffffffu, staged[base + lane] == source);
      if (match) { found = base + static_cast<uint32_t>(__ffs(match)) - 1u; break; }
    }
    const uint8_t* from = found != 0xffffffffu
                              ? view.staging + (static_cast<uint64_t>(b) * view.capacity + found) * a.tokenBytes
                              : a.source_base + source;
    served += found != 0xffffffffu;
    copy_row(a.pool + static_cast<uint64_t>(dest) * a.tokenBytes, from, a.tokenBytes, lane);
    if (lane == 0 && slot < a.resident) a.hot_valid[static_cast<uint64_t>(owner) * a.resident + slot] = 1;
  }
  if (lane == 0 && served && view.hits) atomicAdd(view.hits + b, static_cast<int32_t>(served));
}

}  // namespace

uint32_t launch_fetch_staged(const KvipFetchArgs& a, const KvipWorkspace& ws, cudaStream_t stream) {
  KVIP_REQUIRE(ws.staged_sources && ws.staged_rows && ws.staging && ws.staged_capacity >= 1 &&
                   ws.staged_capacity <= kStagedMax, "fetch: the staging area is not fully described");
  StagedView view{reinterpret_cast<const int64_t*>(static_cast<uintptr_t>(ws.staged_sources)),
                  reinterpret_cast<const int32_t*>(static_cast<uintptr_t>(ws.staged_rows)),
                  reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(ws.staging)),
                  reinterpret_cast<int32_t*>(static_cast<uintptr_t>(ws.staged_hits)), ws.staged_capacity};
  dim3 grid(kFetchBlocksPerRequest, a.batch);
  fetch_rows_staged<<<grid, kFetchThreads, 0, stream>>>(a, view);
  count_launch();
  return check_launch("fetch_rows_staged");
}

}  // namespace kvip

extern "C" uint32_t kvip_b200_window_bounds(const KvipWindowArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->key_lengths && a->query_ends && a->window_lengths && a->window_ends && a->staged_count &&
                   a->staged_rows, "window_bounds: null pointer");
  KVIP_REQUIRE(a->batch >= 1 && a->queries >= 1 && a->queries <= KVIP_MAX_QUERIES && a->windows >= 1 && a->windows <= 8,
               "window_bounds: geometry");
  for (uint32_t w = 0; w < a->windows; ++w)
    KVIP_REQUIRE(a->first[w] < a->first[w + 1] && a->first[w] % KVIP_BLOCK_TOKENS == 0,
                 "window_bounds: windows are increasing and start on a key page");
  const uint32_t items = a->windows * a->batch * a->queries;
  kvip::window_bounds<<<(items + 255u) / 256u, 256, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("window_bounds");
}

extern "C" uint32_t kvip_b200_resident_threshold(const KvipThresholdArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->prefix_topk && a->prefix_scores && a->thresholds && a->rows >= 1, "resident_threshold: arguments");
  kvip::resident_threshold<<<a->rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  kvip::count_launch();
  return kvip::check_launch("resident_threshold");
}

extern "C" uint32_t kvip_b200_speculate_window(const KvipSpeculateArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->scores && a->thresholds && a->key_lengths && a->query_ends && a->addresses && a->source_base &&
                   a->staged_sources && a->staged_count && a->staged_rows && a->staging, "speculate_window: null pointer");
  KVIP_REQUIRE(a->batch >= 1 && a->queries >= 1 && a->queries <= KVIP_MAX_QUERIES && a->first < a->last &&
                   a->last <= a->scoreStride, "speculate_window: geometry");
  KVIP_REQUIRE(a->capacity >= 1 && a->capacity <= kvip::kStagedMax && a->limit <= a->capacity,
               "speculate_window: at most 512 staged rows per request");
  KVIP_REQUIRE(a->tokenBytes >= 16 && a->tokenBytes % 16 == 0, "speculate_window: rows are multiples of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((a->last - a->first + 255u) / 256u, a->batch);
  kvip::speculate_collect<<<grid, 256, 0, s>>>(*a);
  uint32_t rc = kvip::check_launch("speculate_collect");
  if (rc) return rc;
  kvip::speculate_copy<<<a->batch, 512, 0, s>>>(*a);
  kvip::count_launch(2);
  return kvip::check_launch("speculate_copy");
}
