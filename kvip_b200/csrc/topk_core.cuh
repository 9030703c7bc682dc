// Shared pieces of the TopK kernels: the warp-aggregated histogram update and the single-CTA selection
// of one score row (used by topk.cu directly and by topk_split.cu for rows whose threshold bin overflows).
#pragma once
#include "common.cuh"

namespace kvip {
namespace topk_core {

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

constexpr uint32_t kCandidates = 8192;  // shared-memory candidates of the threshold bin

// The whole selection of one row by one CTA of kThreads threads. `global_hist` is the row's 12-bit
// histogram in global memory (consumed and cleared) or NULL (the first pass is then done here).
static __device__ void select_row(const KvipTopkArgs& a, const uint32_t row, uint32_t* global_hist) {
  __shared__ uint32_t hist[4096];
  __shared__ uint32_t scan_scratch[33];
  __shared__ uint32_t found[2];
  __shared__ uint32_t cand_count;
  extern __shared__ uint32_t cand_keys[];  // [kCandidates] when a histogram is supplied
  const uint32_t tid = threadIdx.x;
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
    if (pass == 0 && global_hist) {
      for (uint32_t i = tid; i < bins; i += kThreads) { hist[i] = global_hist[i]; global_hist[i] = 0; }
      if (tid == 0) cand_count = 0;
    } else {
      for (uint32_t i = tid; i < bins; i += kThreads) hist[i] = 0;
    }
    if (tid == 0) { found[0] = 0; found[1] = 0; }   // defined even when a supplied histogram was inconsistent
    __syncthreads();
    // every lane of a warp runs the same number of iterations (hist_add uses warp votes)
    const uint32_t rounds = (pass == 0 && global_hist) ? 0u : (in_smem ? (cand_count + kThreads - 1) / kThreads
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
    if (pass == 0 && global_hist) {
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
            if ((v * 4u + j) < L && (key & prefix_mask) == prefix) {
              // the bound holds whenever the histogram told the truth; a histogram that undercounted the bin
              // (a caller's scratch that was not all-zero, two calls racing on one scratch) must not write
              // past the list: the count then exceeds the capacity and the global passes take over
              const uint32_t at = atomicAdd(&cand_count, 1u);
              if (at < kCandidates) cand_keys[at] = key;
            }
          }
        }
      }
      __syncthreads();
      in_smem = want <= kCandidates && cand_count <= kCandidates;   // block-uniform
      __syncthreads();
    }
  }
  const uint32_t kth = prefix;             // exact key of the 2048th largest element
  const uint32_t need_eq = remaining;      // how many == kth positions are taken
  const uint32_t count_gt = kTop - need_eq;

  // ordered compaction: every warp owns a contiguous run of the chunk (coalesced 128-byte loads), the rank of
  // a winner inside a group of 32 positions comes from a ballot, one block scan per chunk orders the warps
  uint32_t gt_base = 0, eq_base = 0;
  const uint32_t lane = tid & 31u, warp = tid >> 5, below = (1u << lane) - 1u;
  constexpr uint32_t kGroups = kItems;                  // groups of 32 positions per warp and chunk
  const uint32_t chunk = kThreads * kGroups;
  for (uint32_t start = 0; start < L; start += chunk) {
    const uint32_t run = start + warp * (32u * kGroups);
    float e[kGroups];
    uint32_t warp_gt = 0, warp_eq = 0;
#pragma unroll
    for (uint32_t j = 0; j < kGroups; ++j) {
      const uint32_t position = run + j * 32u + lane;
      e[j] = position < L ? scores[position] : 0.f;
      const uint32_t key = sortable_key(e[j]);
      warp_gt += __popc(__ballot_sync(0xffffffffu, position < L && key > kth));
      warp_eq += __popc(__ballot_sync(0xffffffffu, position < L && key == kth));
    }
    uint32_t total;
    uint32_t offset = block_exclusive_scan(lane == 0 ? (warp_gt | (warp_eq << 16)) : 0u, scan_scratch, &total);
    offset = __shfl_sync(0xffffffffu, offset, 0);
    uint32_t g = gt_base + (offset & 0xffffu), q = eq_base + (offset >> 16);
#pragma unroll
    for (uint32_t j = 0; j < kGroups; ++j) {
      const uint32_t position = run + j * 32u + lane;
      const uint32_t key = sortable_key(e[j]);
      const uint32_t mask_gt = __ballot_sync(0xffffffffu, position < L && key > kth);
      const uint32_t mask_eq = __ballot_sync(0xffffffffu, position < L && key == kth);
      if ((mask_gt >> lane) & 1u) {
        const uint32_t at = g + __popc(mask_gt & below);
        if (at < kTop) {   // always true for a consistent selection; keeps a corrupted scratch from writing past the row
          out[at] = static_cast<int32_t>(position + a.base_index);
          if (out_scores) out_scores[at] = e[j];
        }
      } else if ((mask_eq >> lane) & 1u) {
        const uint32_t rank = q + __popc(mask_eq & below);
        if (rank < need_eq && count_gt + rank < kTop) {
          out[count_gt + rank] = static_cast<int32_t>(position + a.base_index);
          if (out_scores) out_scores[count_gt + rank] = e[j];
        }
      }
      g += __popc(mask_gt);
      q += __popc(mask_eq);
    }
    gt_base += total & 0xffffu;
    eq_base += total >> 16;
    if (gt_base == count_gt && eq_base >= need_eq) break;  // block-uniform
  }
}

}  // namespace topk_core
}  // namespace kvip
