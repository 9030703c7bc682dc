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
// One CTA per query row. Three histogram passes (12 + 12 + 8 bits of the order-preserving
// u32 image of the float) find v exactly; a fourth, ordered pass compacts the winners with
// block-wide prefix sums (no atomics, so the order is the position order). The row is read
// from L2 (the LI kernel has just written it) with 16-byte loads.
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kThreads = 1024;
constexpr uint32_t kItems = 16;  // consecutive elements per thread in the ordered pass

__device__ __forceinline__ void hist_add(uint32_t* hist, bool valid, uint32_t bin) {
  // Degenerate rows (every lane in one bin, e.g. an all-zero score row) would serialise
  // on one shared-memory word: one lane adds for the whole warp instead.
  const uint32_t first = __shfl_sync(0xffffffffu, bin, 0);
  if (__all_sync(0xffffffffu, valid && bin == first)) {
    if ((threadIdx.x & 31u) == 0) atomicAdd(hist + first, 32u);
  } else if (valid) {
    atomicAdd(hist + bin, 1u);
  }
}

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

constexpr uint32_t kCandidates = 8192;  // shared-memory candidates of the threshold bin

__global__ void __launch_bounds__(kThreads) topk_select(const KvipTopkArgs a) {
  __shared__ uint32_t hist[4096];
  __shared__ uint32_t scan_scratch[33];
  __shared__ uint32_t found[2];
  __shared__ uint32_t cand_count;
  extern __shared__ uint32_t cand_keys[];  // [kCandidates] when a histogram is supplied
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  const uint32_t b = row / a.queries;
  int32_t valid_len = min(a.key_lengths[b], a.query_ends[row]);
  valid_len = min(valid_len, static_cast<int32_t>(a.scoreStride));
  int32_t* out = a.topk + static_cast<uint64_t>(row) * kTop;
  float* out_scores = a.topk_scores ? a.topk_scores + static_cast<uint64_t>(row) * kTop : nullptr;
  const float* scores = a.scores + static_cast<uint64_t>(row) * a.scoreStride;
  if (valid_len <= static_cast<int32_t>(kTop)) {
    for (uint32_t i = tid; i < kTop; i += kThreads) {
      const bool live = static_cast<int32_t>(i) < valid_len;
      out[i] = live ? static_cast<int32_t>(i + a.base_index) : -1;
      if (out_scores) out_scores[i] = live ? scores[i] : 0.f;
    }
    return;
  }
  const uint32_t L = static_cast<uint32_t>(valid_len);
  const uint32_t vec_count = (L + 3u) >> 2;
  const float4* row4 = reinterpret_cast<const float4*>(scores);

  uint32_t prefix = 0, prefix_mask = 0, remaining = kTop;
  bool in_smem = false;  // passes 2 and 3 run over the shared-memory candidates instead of the row
#pragma unroll 1
  for (uint32_t pass = 0; pass < 3; ++pass) {
    const uint32_t bits = pass == 2 ? 8u : 12u;
    const uint32_t shift = pass == 0 ? 20u : (pass == 1 ? 8u : 0u);
    const uint32_t bins = 1u << bits;
    if (pass == 0 && a.histogram) {
      uint32_t* global_hist = a.histogram + static_cast<uint64_t>(row) * 4096u;
      for (uint32_t i = tid; i < bins; i += kThreads) { hist[i] = global_hist[i]; global_hist[i] = 0; }
      if (tid == 0) cand_count = 0;
    } else {
      for (uint32_t i = tid; i < bins; i += kThreads) hist[i] = 0;
    }
    __syncthreads();
    // every lane of a warp runs the same number of iterations (hist_add uses warp votes)
    const uint32_t rounds = (pass == 0 && a.histogram) ? 0u : (in_smem ? (cand_count + kThreads - 1) / kThreads
                                                                       : (vec_count + kThreads - 1) / kThreads);
    if (in_smem) {
      const uint32_t n = cand_count;
      for (uint32_t r = 0; r < rounds; ++r) {
        const uint32_t i = r * kThreads + tid;
        const uint32_t key = i < n ? cand_keys[i] : 0u;
        hist_add(hist, i < n && (key & prefix_mask) == prefix, (key >> shift) & (bins - 1u));
      }
    } else
    for (uint32_t r = 0; r < rounds; ++r) {
      const uint32_t v = r * kThreads + tid;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (v < vec_count) x = row4[v];
      const float e[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        const uint32_t key = sortable_key(e[j]);
        const bool ok = v < vec_count && (v * 4u + j) < L && (key & prefix_mask) == prefix;
        hist_add(hist, ok, (key >> shift) & (bins - 1u));
      }
    }
    __syncthreads();
    // thread i owns the 4 (or fewer) highest unclaimed bins: suffix counts via a scan over
    // reversed bin groups
    const uint32_t per = bins / kThreads ? bins / kThreads : 1u;  // 4, 4, then 1 (256 bins)
    const uint32_t groups = bins / per;
    uint32_t local = 0;
    const uint32_t group = groups - 1u - tid;  // valid when tid < groups
    if (tid < groups)
      for (uint32_t j = 0; j < per; ++j) local += hist[group * per + j];
    uint32_t above = block_exclusive_scan(local, scan_scratch, nullptr);
    if (tid < groups) {
      for (int32_t j = static_cast<int32_t>(per) - 1; j >= 0; --j) {
        const uint32_t bin = group * per + static_cast<uint32_t>(j);
        const uint32_t c = hist[bin];
        if (above < remaining && above + c >= remaining) {
          found[0] = bin;
          found[1] = remaining - above;
        }
        above += c;
      }
    }
    __syncthreads();
    prefix |= found[0] << shift;
    prefix_mask |= (bins - 1u) << shift;
    remaining = found[1];
    __syncthreads();
    if (pass == 0 && a.histogram) {
      // One cheap pass collects the threshold bin's keys; if they fit, the remaining 20 bits are
      // resolved in shared memory. (An overfull bin, e.g. a constant row, keeps the global passes.)
      const uint32_t want = hist[prefix >> 20];
      if (want <= kCandidates) {
        const uint32_t rounds_f = (vec_count + kThreads - 1) / kThreads;
        for (uint32_t r = 0; r < rounds_f; ++r) {
          const uint32_t v = r * kThreads + tid;
          if (v >= vec_count) continue;
          const float4 x = row4[v];
          const float e[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t key = sortable_key(e[j]);
            if ((v * 4u + j) < L && (key & prefix_mask) == prefix) cand_keys[atomicAdd(&cand_count, 1u)] = key;
          }
        }
        in_smem = true;
      }
      __syncthreads();
    }
  }
  const uint32_t kth = prefix;             // exact key of the 2048th largest element
  const uint32_t need_eq = remaining;      // how many == kth positions are taken
  const uint32_t count_gt = kTop - need_eq;

  // ordered compaction
  uint32_t gt_base = 0, eq_base = 0;
  const uint32_t chunk = kThreads * kItems;
  for (uint32_t start = 0; start < L; start += chunk) {
    const uint32_t first = start + tid * kItems;
    float e[kItems];
    uint32_t flags_gt = 0, flags_eq = 0;
#pragma unroll
    for (uint32_t v = 0; v < kItems / 4; ++v) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (first + v * 4u < L) x = row4[(first >> 2) + v];
      e[v * 4 + 0] = x.x; e[v * 4 + 1] = x.y; e[v * 4 + 2] = x.z; e[v * 4 + 3] = x.w;
    }
#pragma unroll
    for (uint32_t j = 0; j < kItems; ++j) {
      const uint32_t key = sortable_key(e[j]);
      const bool live = first + j < L;
      flags_gt |= (live && key > kth ? 1u : 0u) << j;
      flags_eq |= (live && key == kth ? 1u : 0u) << j;
    }
    const uint32_t packed = __popc(flags_gt) | (__popc(flags_eq) << 16);
    uint32_t total;
    const uint32_t offset = block_exclusive_scan(packed, scan_scratch, &total);
    uint32_t g = gt_base + (offset & 0xffffu), q = eq_base + (offset >> 16);
#pragma unroll
    for (uint32_t j = 0; j < kItems; ++j) {
      if ((flags_gt >> j) & 1u) {
        out[g] = static_cast<int32_t>(first + j + a.base_index);
        if (out_scores) out_scores[g] = e[j];
        ++g;
      } else if ((flags_eq >> j) & 1u) {
        if (q < need_eq) {
          out[count_gt + q] = static_cast<int32_t>(first + j + a.base_index);
          if (out_scores) out_scores[count_gt + q] = e[j];
        }
        ++q;
      }
    }
    gt_base += total & 0xffffu;
    eq_base += total >> 16;
    if (gt_base == count_gt && eq_base >= need_eq) break;  // block-uniform
  }
}

// ---- merge of shard candidates -----------------------------------------------------------
// Bitonic sort of (key descending, index ascending) composites in shared memory, cut at
// 2048, then a second sort that restores the canonical output order.
__device__ __forceinline__ void bitonic_sort(uint64_t* data, uint32_t n) {
  for (uint32_t k = 2; k <= n; k <<= 1) {
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t partner = i ^ j;
        if (partner > i) {
          const uint64_t x = data[i], y = data[partner];
          const bool ascending = (i & k) == 0;
          if ((x > y) == ascending) { data[i] = y; data[partner] = x; }
        }
      }
      __syncthreads();
    }
  }
}

__global__ void __launch_bounds__(kThreads) topk_merge(const KvipMergeArgs a, uint32_t padded) {
  extern __shared__ uint64_t composite[];
  const uint32_t row = blockIdx.x, n = a.shards * kTop;
  const float* cs = a.cand_scores + static_cast<uint64_t>(row) * n;
  const int32_t* ci = a.cand_index + static_cast<uint64_t>(row) * n;
  for (uint32_t i = threadIdx.x; i < padded; i += kThreads) {
    uint64_t c = ~0ull;
    if (i < n && ci[i] >= 0)
      c = (static_cast<uint64_t>(~sortable_key(cs[i])) << 32) | static_cast<uint32_t>(ci[i]);
    composite[i] = c;
  }
  __syncthreads();
  bitonic_sort(composite, padded);
  // canonical order: keys above the cut by ascending index, then the cut key by ascending index
  const uint32_t cut_key = static_cast<uint32_t>(composite[kTop - 1] >> 32);
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < kTop; i += kThreads) {
    const uint64_t c = composite[i];
    if (c != ~0ull) {
      const uint64_t tie = static_cast<uint32_t>(c >> 32) == cut_key ? 1ull : 0ull;
      composite[i] = (tie << 32) | (c & 0xffffffffull);
    }
  }
  __syncthreads();
  bitonic_sort(composite, kTop);
  int32_t* out = a.topk + static_cast<uint64_t>(row) * kTop;
  for (uint32_t i = threadIdx.x; i < kTop; i += kThreads)
    out[i] = composite[i] == ~0ull ? -1 : static_cast<int32_t>(composite[i] & 0xffffffffull);
}

}  // namespace

uint32_t launch_topk(const KvipTopkArgs& a, cudaStream_t stream) {
  size_t smem = 0;
  if (a.histogram) {
    uint32_t segments = (4u * 148u + a.rows - 1u) / a.rows;
    segments = segments < 1u ? 1u : (segments > 32u ? 32u : segments);
    topk_histogram<<<dim3(segments, a.rows), kHistThreads, 0, stream>>>(a);
    count_launch();
    if (uint32_t bad = check_launch("topk_histogram")) return bad;
    smem = kCandidates * sizeof(uint32_t);
    static bool configured = false;  // static + dynamic shared memory exceeds the 48 KiB default
    if (!configured) {
      if (cudaFuncSetAttribute(topk_select, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess)
        return check_launch("topk_select attribute");
      configured = true;
    }
  }
  topk_select<<<a.rows, kThreads, smem, stream>>>(a);
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
  return kvip::launch_topk(with_scratch, s);
}

extern "C" uint32_t kvip_b200_topk_merge(const KvipMergeArgs* a, void* stream) {
  KVIP_REQUIRE(a && a->cand_scores && a->cand_index && a->topk, "topk_merge: null pointer");
  KVIP_REQUIRE(a->rows >= 1 && a->shards >= 1 && a->shards <= 8, "topk_merge: 1..8 shards");
  uint32_t padded = 2048;
  while (padded < a->shards * KVIP_TOPK) padded <<= 1;
  const size_t smem = static_cast<size_t>(padded) * sizeof(uint64_t);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kvip::topk_merge, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 8) != cudaSuccess)
      return kvip::check_launch("topk_merge attribute");
    configured = true;
  }
  kvip::topk_merge<<<a->rows, kvip::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(*a, padded);
  kvip::count_launch();
  return kvip::check_launch("topk_merge");
}
