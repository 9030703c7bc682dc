// TopK-2048 with every pass spread over the whole GPU.
//
// A decode batch has far fewer score rows (64) than the GPU has SMs (148), and one CTA can only pull a
// fraction of the L2 bandwidth, so the one-CTA-per-row selection leaves most of the machine idle. Here
// each row is cut into `segments` contiguous slices and every pass runs on segments x rows CTAs:
//
//   1. split_histogram  12-bit histogram of the order-preserving keys -> row histogram (global atomics)
//   2. split_filter     every CTA finds the threshold bin from the row histogram, counts its slice's
//                       keys in higher bins and appends the threshold bin's (key, position) pairs to
//                       the row's candidate list
//   3. split_emit       every CTA resolves the exact 2048th key from the candidate list in shared
//                       memory, derives how many winners lie in earlier slices (higher-bin counts +
//                       candidates) and writes its slice's winners at their final positions
//   4. split_fallback   rows whose threshold bin holds more than 8192 keys (constant rows) are
//                       selected by the single-CTA kernel instead
//
// The output is the same canonical order as the single-CTA kernel (positions with key > v ascending,
// then key == v ascending): offsets come from prefix sums over slices and threads, never from arrival
// order. The scratch row is handed back all-zero.
#include "common.cuh"
#include "topk_core.cuh"

namespace kvip {
namespace {

using topk_core::hist_add;
using topk_core::kCandidates;
constexpr uint32_t kSplitThreads = 512;
constexpr uint32_t kMaxSegments = 32;
constexpr uint32_t kHeader = 64;                      // words after the histogram
constexpr uint32_t kSegAbove = 4096, kCandCount = 4096 + 32, kDone = 4096 + 33, kOverflow = 4096 + 34;
constexpr uint32_t kCandKeys = 4096 + kHeader, kCandIndex = kCandKeys + kCandidates;
constexpr uint32_t kRowWords = kCandIndex + kCandidates;  // == KVIP_TOPK_SPLIT_WORDS
static_assert(kRowWords == KVIP_TOPK_SPLIT_WORDS, "scratch row size is part of the ABI");
constexpr uint32_t kMaxGroups = 36;  // groups of 32 positions one warp of split_emit compacts

struct Slice {
  uint32_t length, vec_count, per_vec, begin_vec, end_vec;
};

__device__ __forceinline__ bool slice_of(const KvipTopkArgs& a, uint32_t row, uint32_t segment, uint32_t segments,
                                         Slice* s) {
  int32_t valid_len = min(a.key_lengths[row / a.queries], a.query_ends[row]);
  valid_len = min(valid_len, static_cast<int32_t>(a.scoreStride));
  if (valid_len <= static_cast<int32_t>(kTop)) { s->length = static_cast<uint32_t>(max(valid_len, 0)); return false; }
  s->length = static_cast<uint32_t>(valid_len);
  s->vec_count = (s->length + 3u) >> 2;
  s->per_vec = ((s->vec_count + segments - 1u) / segments + 255u) / 256u * 256u;  // float4s per slice
  s->begin_vec = min(segment * s->per_vec, s->vec_count);
  s->end_vec = min(s->begin_vec + s->per_vec, s->vec_count);
  return true;
}

// Threshold bin of a 4096-bin histogram in shared memory: the bin where the count from the top reaches
// 2048. Returns the bin; *above receives the number of keys in higher bins.
__device__ __forceinline__ uint32_t threshold_bin(const uint32_t* hist, uint32_t* scan, uint32_t* found, uint32_t* above_out) {
  constexpr uint32_t per = 4096 / kSplitThreads;
  const uint32_t group = kSplitThreads - 1u - threadIdx.x;
  uint32_t local = 0;
#pragma unroll
  for (uint32_t j = 0; j < per; ++j) local += hist[group * per + j];
  uint32_t above = block_exclusive_scan(local, scan, nullptr);
  for (int32_t j = per - 1; j >= 0; --j) {
    const uint32_t c = hist[group * per + j];
    if (above < kTop && above + c >= kTop) { found[0] = group * per + j; found[1] = above; }
    above += c;
  }
  __syncthreads();
  *above_out = found[1];
  return found[0];
}

__global__ void __launch_bounds__(kSplitThreads) split_histogram(const KvipTopkArgs a) {
  __shared__ uint32_t hist[4096];
  const uint32_t row = blockIdx.y, tid = threadIdx.x;
  Slice s;
  if (!slice_of(a, row, blockIdx.x, gridDim.x, &s) || s.begin_vec >= s.end_vec) return;
  for (uint32_t i = tid; i < 4096; i += kSplitThreads) hist[i] = 0;
  __syncthreads();
  const float4* row4 = reinterpret_cast<const float4*>(a.scores + static_cast<uint64_t>(row) * a.scoreStride);
  for (uint32_t v0 = s.begin_vec; v0 < s.end_vec; v0 += kSplitThreads) {
    const uint32_t v = v0 + tid;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (v < s.end_vec) x = row4[v];
    const float e[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) hist_add(hist, v < s.end_vec && (v * 4u + j) < s.length, sortable_key(e[j]) >> 20);
  }
  __syncthreads();
  uint32_t* out = a.split_scratch + static_cast<uint64_t>(row) * kRowWords;
  for (uint32_t i = tid; i < 4096; i += kSplitThreads)
    if (hist[i]) atomicAdd(out + i, hist[i]);
}

__global__ void __launch_bounds__(kSplitThreads) split_filter(const KvipTopkArgs a) {
  __shared__ uint32_t hist[4096];
  __shared__ uint32_t scan[33];
  __shared__ uint32_t found[2];
  __shared__ uint32_t above_total;
  const uint32_t row = blockIdx.y, tid = threadIdx.x;
  Slice s;
  if (!slice_of(a, row, blockIdx.x, gridDim.x, &s)) return;
  uint32_t* scratch = a.split_scratch + static_cast<uint64_t>(row) * kRowWords;
  for (uint32_t i = tid; i < 4096; i += kSplitThreads) hist[i] = scratch[i];
  if (tid == 0) above_total = 0;
  __syncthreads();
  uint32_t unused;
  const uint32_t bin = threshold_bin(hist, scan, found, &unused);
  const float4* row4 = reinterpret_cast<const float4*>(a.scores + static_cast<uint64_t>(row) * a.scoreStride);
  uint32_t above = 0;
  for (uint32_t v = s.begin_vec + tid; v < s.end_vec; v += kSplitThreads) {
    const float4 x = row4[v];
    const float e[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
      const uint32_t position = v * 4u + j;
      if (position >= s.length) continue;
      const uint32_t key = sortable_key(e[j]), b = key >> 20;
      if (b > bin) {
        ++above;
      } else if (b == bin) {
        const uint32_t slot = atomicAdd(scratch + kCandCount, 1u);
        if (slot < kCandidates) { scratch[kCandKeys + slot] = key; scratch[kCandIndex + slot] = position; }
      }
    }
  }
#pragma unroll
  for (uint32_t o = 16; o > 0; o >>= 1) above += __shfl_xor_sync(0xffffffffu, above, o);
  if ((tid & 31u) == 0 && above) atomicAdd(&above_total, above);
  __syncthreads();
  if (tid == 0) scratch[kSegAbove + blockIdx.x] = above_total;
}

__global__ void __launch_bounds__(kSplitThreads) split_emit(const KvipTopkArgs a) {
  extern __shared__ uint32_t smem[];
  uint32_t* cand_key = smem;                      // [kCandidates]
  uint32_t* cand_pos = smem + kCandidates;        // [kCandidates]
  uint32_t* hist = cand_pos + kCandidates;        // [1024]
  uint32_t* scan = hist + 1024;                   // [33]
  uint32_t* shared = scan + 33;                   // [8]: 0 digit, 1 remaining, 2..4 block sums, 5 last flag
  const uint32_t row = blockIdx.y, segment = blockIdx.x, segments = gridDim.x, tid = threadIdx.x;
  int32_t* out = a.topk + static_cast<uint64_t>(row) * kTop;
  float* out_scores = a.topk_scores ? a.topk_scores + static_cast<uint64_t>(row) * kTop : nullptr;
  const float* scores = a.scores + static_cast<uint64_t>(row) * a.scoreStride;
  Slice s;
  if (!slice_of(a, row, segment, segments, &s)) {
    if (segment == 0)
      for (uint32_t i = tid; i < kTop; i += kSplitThreads) {
        const bool live = i < s.length;
        out[i] = live ? static_cast<int32_t>(i + a.base_index) : -1;
        if (out_scores) out_scores[i] = live ? scores[i] : 0.f;
      }
    return;
  }
  uint32_t* scratch = a.split_scratch + static_cast<uint64_t>(row) * kRowWords;
  const uint32_t n = scratch[kCandCount];
  const bool overflow = n > kCandidates;
  if (!overflow) {
    uint32_t total_above = 0, above_before = 0;
    for (uint32_t i = 0; i < segments; ++i) {
      const uint32_t c = scratch[kSegAbove + i];
      total_above += c;
      if (i < segment) above_before += c;
    }
    for (uint32_t i = tid; i < n; i += kSplitThreads) { cand_key[i] = scratch[kCandKeys + i]; cand_pos[i] = scratch[kCandIndex + i]; }
    // exact 2048th key: two 10-bit passes over the candidates' low 20 bits
    uint32_t remaining = kTop - total_above, low = 0, low_mask = 0;
    for (uint32_t pass = 0; pass < 2; ++pass) {
      const uint32_t shift = pass ? 0u : 10u;
      for (uint32_t i = tid; i < 1024; i += kSplitThreads) hist[i] = 0;
      __syncthreads();
      const uint32_t rounds = (n + kSplitThreads - 1u) / kSplitThreads;
      for (uint32_t r = 0; r < rounds; ++r) {
        const uint32_t i = r * kSplitThreads + tid;
        const uint32_t key = i < n ? cand_key[i] & 0xfffffu : 0u;
        hist_add(hist, i < n && (key & low_mask) == low, (key >> shift) & 1023u);
      }
      __syncthreads();
      const uint32_t group = kSplitThreads - 1u - tid;  // two bins per thread, highest first
      uint32_t above = block_exclusive_scan(hist[group * 2u] + hist[group * 2u + 1u], scan, nullptr);
      for (int32_t j = 1; j >= 0; --j) {
        const uint32_t c = hist[group * 2u + j];
        if (above < remaining && above + c >= remaining) { shared[0] = group * 2u + j; shared[1] = remaining - above; }
        above += c;
      }
      __syncthreads();
      low |= shared[0] << shift;
      low_mask |= 1023u << shift;
      remaining = shared[1];
      __syncthreads();
    }
    const uint32_t bin = n ? cand_key[0] >> 20 : 0u;
    const uint32_t kth = (bin << 20) | low;
    const uint32_t need_eq = remaining;
    // winners among the candidates that lie in earlier slices, and candidates above the cut in total
    const uint32_t slice_elems = s.per_vec * 4u;
    uint32_t gt_before = 0, eq_before = 0, gt_cand = 0;
    for (uint32_t i = tid; i < n; i += kSplitThreads) {
      const uint32_t key = cand_key[i];
      const bool earlier = cand_pos[i] / slice_elems < segment;
      if (key > kth) { ++gt_cand; gt_before += earlier; }
      else if (key == kth) eq_before += earlier;
    }
    if (tid < 3) shared[2 + tid] = 0;
    __syncthreads();
#pragma unroll
    for (uint32_t o = 16; o > 0; o >>= 1) {
      gt_before += __shfl_xor_sync(0xffffffffu, gt_before, o);
      eq_before += __shfl_xor_sync(0xffffffffu, eq_before, o);
      gt_cand += __shfl_xor_sync(0xffffffffu, gt_cand, o);
    }
    if ((tid & 31u) == 0) { atomicAdd(shared + 2, gt_before); atomicAdd(shared + 3, eq_before); atomicAdd(shared + 4, gt_cand); }
    __syncthreads();
    const uint32_t count_gt = total_above + shared[4];
    uint32_t gt_base = above_before + shared[2], eq_base = shared[3];
    // ordered compaction of this slice: every warp owns a contiguous run (coalesced 128-byte loads), ranks
    // inside a group of 32 come from ballots, one block scan orders the warps
    const uint32_t slice_begin = s.begin_vec * 4u, slice_end = min(s.end_vec * 4u, s.length);
    const uint32_t lane = tid & 31u, warp = tid >> 5, warps = kSplitThreads / 32u;
    const uint32_t groups = (slice_end - slice_begin + 31u) / 32u;          // groups of 32 positions
    const uint32_t per_warp = (groups + warps - 1u) / warps;                // <= kMaxGroups
    const uint32_t run_begin = slice_begin + warp * per_warp * 32u;
    float value[kMaxGroups];  // the ballots are recomputed when writing: only the values stay in registers
    uint32_t warp_gt = 0, warp_eq = 0;
#pragma unroll
    for (uint32_t j = 0; j < kMaxGroups; ++j) {
      const uint32_t position = run_begin + j * 32u + lane;
      const bool live = j < per_warp && position < slice_end;
      value[j] = live ? scores[position] : 0.f;
      const uint32_t key = sortable_key(value[j]);
      warp_gt += __popc(__ballot_sync(0xffffffffu, live && key > kth));
      warp_eq += __popc(__ballot_sync(0xffffffffu, live && key == kth));
    }
    uint32_t offset = block_exclusive_scan(lane == 0 ? (warp_gt | (warp_eq << 16)) : 0u, scan, nullptr);
    offset = __shfl_sync(0xffffffffu, offset, 0);
    uint32_t g = gt_base + (offset & 0xffffu), q = eq_base + (offset >> 16);
    const uint32_t below = (1u << lane) - 1u;
#pragma unroll
    for (uint32_t j = 0; j < kMaxGroups; ++j) {
      const uint32_t position = run_begin + j * 32u + lane;
      const bool live = j < per_warp && position < slice_end;
      const uint32_t key = sortable_key(value[j]);
      const uint32_t mask_gt = __ballot_sync(0xffffffffu, live && key > kth);
      const uint32_t mask_eq = __ballot_sync(0xffffffffu, live && key == kth);
      if ((mask_gt >> lane) & 1u) {
        const uint32_t at = g + __popc(mask_gt & below);
        out[at] = static_cast<int32_t>(position + a.base_index);
        if (out_scores) out_scores[at] = value[j];
      } else if ((mask_eq >> lane) & 1u) {
        const uint32_t rank = q + __popc(mask_eq & below);
        if (rank < need_eq) {
          out[count_gt + rank] = static_cast<int32_t>(position + a.base_index);
          if (out_scores) out_scores[count_gt + rank] = value[j];
        }
      }
      g += __popc(mask_gt);
      q += __popc(mask_eq);
    }
  }
  // the last CTA of the row hands the scratch back all-zero (an overflowing row keeps its histogram for
  // the fallback kernel, which clears it)
  __threadfence();
  __syncthreads();
  if (tid == 0) shared[5] = atomicAdd(scratch + kDone, 1u) == segments - 1u ? 1u : 0u;
  __syncthreads();
  if (shared[5]) {
    if (!overflow)
      for (uint32_t i = tid; i < 4096; i += kSplitThreads) scratch[i] = 0;
    for (uint32_t i = tid; i < kHeader; i += kSplitThreads) scratch[4096 + i] = (overflow && 4096 + i == kOverflow) ? 1u : 0u;
  }
}

__global__ void __launch_bounds__(topk_core::kThreads) split_fallback(const KvipTopkArgs a) {
  uint32_t* scratch = a.split_scratch + static_cast<uint64_t>(blockIdx.x) * kRowWords;
  if (!scratch[kOverflow]) return;  // block-uniform
  __syncthreads();
  if (threadIdx.x == 0) scratch[kOverflow] = 0;
  topk_core::select_row(a, blockIdx.x, scratch);
}

}  // namespace

uint32_t launch_topk(const KvipTopkArgs& a, cudaStream_t stream);

uint32_t launch_topk_split(const KvipTopkArgs& a, cudaStream_t stream) {
  uint32_t segments = (4u * device_sm_count() + a.rows - 1u) / a.rows;
  segments = segments < 1u ? 1u : (segments > kMaxSegments ? kMaxSegments : segments);
  // a slice must fit the registers of split_emit: 16 warps x kMaxGroups x 32 positions
  const uint32_t slice_limit = (kSplitThreads / 32u) * kMaxGroups * 32u - 1024u;
  while (segments < kMaxSegments && (a.scoreStride + segments - 1u) / segments > slice_limit) ++segments;
  if ((a.scoreStride + segments - 1u) / segments > slice_limit) {  // rows too long to cut into 32 slices
    KvipTopkArgs plain = a;
    plain.split_scratch = nullptr;
    return launch_topk(plain, stream);
  }
  const size_t emit_smem = (2u * kCandidates + 1024u + 33u + 8u) * sizeof(uint32_t);
  const size_t fallback_smem = kCandidates * sizeof(uint32_t);
  if (uint32_t bad = raise_dynamic_smem(kSlotSplitEmit, reinterpret_cast<const void*>(split_emit), 80 * 1024,
                                        "topk split attribute"))
    return bad;
  if (uint32_t bad = raise_dynamic_smem(kSlotSplitFallback, reinterpret_cast<const void*>(split_fallback), 64 * 1024,
                                        "topk split attribute"))
    return bad;
  const dim3 grid(segments, a.rows);
  split_histogram<<<grid, kSplitThreads, 0, stream>>>(a);
  split_filter<<<grid, kSplitThreads, 0, stream>>>(a);
  split_emit<<<grid, kSplitThreads, emit_smem, stream>>>(a);
  split_fallback<<<a.rows, topk_core::kThreads, fallback_smem, stream>>>(a);
  count_launch(4);
  return check_launch("topk split");
}

}  // namespace kvip
