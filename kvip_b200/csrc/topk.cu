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
  const uint64_t shard_stride = a.shard_stride ? a.shard_stride : kTop;
  const uint64_t row_offset = static_cast<uint64_t>(row) * (a.row_stride ? a.row_stride : n);
  for (uint32_t i = threadIdx.x; i < padded; i += kThreads) {
    uint64_t c = ~0ull;
    if (i < n) {
      const uint64_t at = row_offset + (i / kTop) * shard_stride + (i % kTop);
      const int32_t index = a.cand_index[at];
      if (index >= 0) c = (static_cast<uint64_t>(~sortable_key(a.cand_scores[at])) << 32) | static_cast<uint32_t>(index);
    }
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
  KVIP_REQUIRE(a && a->cand_scores && a->cand_index && a->topk, "topk_merge: null pointer");
  KVIP_REQUIRE(a->rows >= 1 && a->shards >= 1 && a->shards <= 8, "topk_merge: 1..8 shards");
  uint32_t padded = 2048;
  while (padded < a->shards * KVIP_TOPK) padded <<= 1;
  const size_t smem = static_cast<size_t>(padded) * sizeof(uint64_t);
  if (uint32_t bad = kvip::raise_dynamic_smem(kvip::kSlotTopkMerge, reinterpret_cast<const void*>(kvip::topk_merge),
                                              16384 * 8, "topk_merge attribute"))
    return bad;
  kvip::topk_merge<<<a->rows, kvip::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(*a, padded);
  kvip::count_launch();
  return kvip::check_launch("topk_merge");
}
