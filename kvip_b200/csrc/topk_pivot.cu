// TopK-2048 of one score row by one CTA (or a pair) that reads the row once: pivot, filter, exact select.
//
// A full radix pass costs one shared-memory atomic per score, and those atomics (not the memory
// traffic) are what a histogram-per-pass selection spends its time on. Here only a SAMPLE of the row
// (128 evenly spaced 128-byte lines per CTA, 4096 scores) goes through a 12-bit histogram. From it a pivot bin
// is chosen that, with a 4-sigma margin, holds at least 2048 keys at or above its lower edge. One
// streaming pass over the row then keeps every score at or above the pivot, in position order, in a
// shared-memory list (ballot + prefix sums, no atomics): typically 3000-6000 of 131072. The exact
// 2048th key is found by the three radix passes (12 + 12 + 8 bits) over that list, and the list is
// emitted in the canonical order stated at the top of topk.cu.
//
// The pivot only has to be safe, not good: the kernel counts what the filter kept, and a row whose list
// would hold fewer than 2048 keys (an unlucky sample) or more than fit (a constant row) is handed to
// the three-passes-over-the-row selection (topk_core::select_row). The result is therefore always the
// exact, deterministic TopK; the sample only decides how fast.
//
// The kernel is instruction-bound (one SM works through a whole row), so while several CTAs per row still fit
// the GPU in one wave it runs as clusters of two, four or eight: each CTA samples and filters its slice of the
// row, rank 0 appends the others' lists through distributed shared memory and finishes alone.
#include <cooperative_groups.h>
#include "common.cuh"
#include "topk_core.cuh"

namespace cg = cooperative_groups;

namespace kvip {
namespace {

using namespace topk_core;

constexpr uint32_t kSampleLines = 128;        // 128-byte lines per CTA that feed the pivot histogram (4096 scores)
constexpr uint32_t kPivotCandidates = 8192;   // capacity of the filtered list (keys + positions: 64 KiB)
constexpr uint32_t kRoundChunks = 8;          // chunks of 16384 scores whose pass masks a thread keeps in registers

__device__ __forceinline__ uint32_t isqrt_ceil(uint32_t v) {
  uint32_t r = static_cast<uint32_t>(sqrtf(static_cast<float>(v)));
  while (r * r < v) ++r;
  return r;
}

__global__ void __launch_bounds__(kThreads, 1) topk_pivot(const KvipTopkArgs a) {
  extern __shared__ uint32_t list[];  // [kPivotCandidates] keys, then [kPivotCandidates] positions
  __shared__ __align__(16) uint32_t hist[4096];
  __shared__ uint32_t scan_scratch[33];
  __shared__ uint32_t found[2];
  __shared__ uint32_t table[kRoundChunks * 32u];  // scores that passed the filter per (chunk, warp) of a round
  __shared__ uint32_t kept_here;                  // what this CTA's filter kept (read by the partner)
  uint32_t* list_key = list;
  uint32_t* list_pos = list + kPivotCandidates;

  // One CTA per row, or a cluster of two, four or eight when the GPU has SMs to spare: each samples and filters
  // its slice of the row, rank 0 appends the others' lists to its own (distributed shared memory) and finishes
  // alone. Every cluster barrier below is reached by all CTAs of the cluster unconditionally.
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t ranks = cluster.num_blocks(), rank = cluster.block_rank();
  const uint32_t row = blockIdx.x / ranks;
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, below = (1u << lane) - 1u;
  const uint32_t b = row / a.queries;
  int32_t valid_len = min(a.key_lengths[b], a.query_ends[row]);
  valid_len = min(valid_len, static_cast<int32_t>(a.scoreStride));
  int32_t* out = a.topk + static_cast<uint64_t>(row) * kTop;
  float* out_scores = a.topk_scores ? a.topk_scores + static_cast<uint64_t>(row) * kTop : nullptr;
  const float* scores = a.scores + static_cast<uint64_t>(row) * a.scoreStride;
  if (valid_len <= static_cast<int32_t>(kTop)) {  // the same for both CTAs of a pair
    if (rank == 0)
    for (uint32_t i = tid; i < kTop; i += kThreads) {
      const bool live = static_cast<int32_t>(i) < valid_len;
      out[i] = live ? static_cast<int32_t>(i + a.base_index) : -1;
      if (out_scores) out_scores[i] = live ? scores[i] : 0.f;
    }
    return;
  }
  const uint32_t L = static_cast<uint32_t>(valid_len);

  // ---- 1. pivot from a sample ------------------------------------------------------------------------
  for (uint32_t i = tid; i < 4096; i += kThreads) hist[i] = 0;
  __syncthreads();
  const uint32_t lines = (L + 31u) >> 5;                       // <= 65536
  const uint32_t sample_lines = min(lines, kSampleLines * ranks);   // every CTA of the cluster samples up to 128 lines
  {
    constexpr uint32_t kPerWarp = kSampleLines / (kThreads / 32u);  // every warp: the same trip count
    float x[kPerWarp];
    bool ok[kPerWarp];
#pragma unroll
    for (uint32_t i = 0; i < kPerWarp; ++i) {  // all loads first: one memory latency, not kPerWarp
      const uint32_t s = (warp + i * (kThreads / 32u)) * ranks + rank;   // sample lines are dealt round-robin
      const uint32_t line = s < sample_lines ? (s * lines) / sample_lines : 0u;
      const uint32_t position = line * 32u + lane;
      ok[i] = s < sample_lines && position < L;
      x[i] = ok[i] ? scores[position] : 0.f;
    }
#pragma unroll
    for (uint32_t i = 0; i < kPerWarp; ++i) hist_add(hist, ok[i], sortable_key(x[i]) >> 20);
  }
  cluster.sync();  // every sample histogram is complete (a block barrier when the cluster is one CTA)
  uint32_t pivot_key;
  {
    const uint32_t group = 1023u - tid;  // thread i owns the 4 highest unclaimed bins
    uint32_t c0 = hist[group * 4u], c1 = hist[group * 4u + 1u], c2 = hist[group * 4u + 2u], c3 = hist[group * 4u + 3u];
    for (uint32_t r = 1; r < ranks; ++r) {
      const uint4 other = *reinterpret_cast<const uint4*>(cluster.map_shared_rank(hist, (rank + r) % ranks) + group * 4u);
      c0 += other.x; c1 += other.y; c2 += other.z; c3 += other.w;
    }
    uint32_t sampled;
    uint32_t above = block_exclusive_scan(c0 + c1 + c2 + c3, scan_scratch, &sampled);
    // expected rank of the 2048th key inside the sample, plus four standard deviations
    uint32_t target = kTop;
    if (sampled < L) {
      const uint32_t mean = static_cast<uint32_t>((static_cast<uint64_t>(kTop) * sampled + L - 1u) / L);
      target = min(sampled, mean + 4u * isqrt_ceil(mean) + 8u);
    }
    const uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
    for (int32_t j = 3; j >= 0; --j) {
      if (above < target && above + c[j] >= target) found[0] = group * 4u + static_cast<uint32_t>(j);
      above += c[j];
    }
    __syncthreads();
    pivot_key = found[0] << 20;
  }

  // ---- 2. one pass over the row: keep key >= pivot, in position order ----------------------------------
  // The filter is instruction-bound (one SM works through the whole row), so the test is one float compare
  // per score: key(x) >= pivot_key  <=>  !(x < pivot_value), except that -0.0 also passes a pivot of +0.0 and
  // everything passes a NaN pivot; a superset is safe, the exact selection below works on keys. A thread owns
  // four 16-byte vectors per chunk of 16384 scores; a warp owns a run of 512 consecutive scores.
  const float pivot_value = __uint_as_float((pivot_key & 0x80000000u) ? (pivot_key ^ 0x80000000u) : ~pivot_key);
  // Two sweeps per round of up to eight chunks (8 x 16384 scores). Sweep A reads the scores and leaves, per
  // thread, only a 16-bit pass mask per chunk (registers) and, per (chunk, warp), the number that passed
  // (shared memory); nothing in it waits for another warp, so the loads of all chunks overlap. One block scan
  // turns the table into list offsets. Sweep B ranks and stores from the masks alone.
  uint32_t kept = 0;  // block-uniform
  {
    const float4* row4 = reinterpret_cast<const float4*>(scores);
    const uint32_t vectors = (L + 3u) >> 2;
    constexpr uint32_t kChunk = kThreads * 16u;
    const uint32_t chunks_each = ((L + kChunk - 1u) / kChunk + ranks - 1u) / ranks;   // rank r: the r-th slice
    const uint32_t begin = min(L, rank * chunks_each * kChunk), end = min(L, (rank + 1u) * chunks_each * kChunk);
    for (uint32_t round = begin; round < end; round += kRoundChunks * kChunk) {
      uint32_t masks[kRoundChunks / 2];
#pragma unroll
      for (uint32_t c = 0; c < kRoundChunks / 2; ++c) masks[c] = 0;
#pragma unroll
      for (uint32_t c = 0; c < kRoundChunks; ++c) {
        const uint32_t start = round + c * kChunk;
        uint32_t mask = 0;
        if (start < end) {  // block-uniform
          const uint32_t run = start + warp * 512u;  // first position of this warp's run
          float4 x[4];
#pragma unroll
          for (uint32_t u = 0; u < 4; ++u) {
            const uint32_t v = (run >> 2) + u * 32u + lane;
            x[u] = v < vectors ? row4[v] : make_float4(0.f, 0.f, 0.f, 0.f);
          }
          const bool tail = start + kChunk > L;  // block-uniform: only the last chunk checks positions
#pragma unroll
          for (uint32_t u = 0; u < 4; ++u) {
            uint32_t bits = (!(x[u].x < pivot_value) ? 1u : 0u) | (!(x[u].y < pivot_value) ? 2u : 0u) |
                            (!(x[u].z < pivot_value) ? 4u : 0u) | (!(x[u].w < pivot_value) ? 8u : 0u);
            if (tail) {
              const uint32_t position = run + u * 128u + lane * 4u;
              bits &= position >= L ? 0u : (L - position >= 4u ? 0xfu : (1u << (L - position)) - 1u);
            }
            mask |= bits << (4u * u);
          }
        }
        masks[c >> 1] |= mask << (16u * (c & 1u));
        const uint32_t passed = __reduce_add_sync(0xffffffffu, __popc(mask));
        if (lane == 0) table[c * 32u + warp] = passed;
      }
      __syncthreads();
      uint32_t total;
      const uint32_t before = block_exclusive_scan(tid < kRoundChunks * 32u ? table[tid] : 0u, scan_scratch, &total);
      if (tid < kRoundChunks * 32u) table[tid] = before;  // (chunk, warp) order is position order
      __syncthreads();
#pragma unroll
      for (uint32_t c = 0; c < kRoundChunks; ++c) {
        uint32_t mask = (masks[c >> 1] >> (16u * (c & 1u))) & 0xffffu;
        if (!__any_sync(0xffffffffu, mask != 0u)) continue;  // nothing of this warp's run passed
        const uint32_t run = round + c * kChunk + warp * 512u;
        // position order inside the run is (vector, lane, element): one warp scan of the four per-vector
        // counts, packed one per byte (at most 128 each: the bytes never carry), ranks all sixteen scores
        const uint32_t packed = __popc(mask & 0xfu) | (__popc(mask & 0xf0u) << 8) | (__popc(mask & 0xf00u) << 16) |
                                (__popc(mask & 0xf000u) << 24);
        uint32_t inclusive = packed;
#pragma unroll
        for (uint32_t d = 1; d < 32; d <<= 1) {
          const uint32_t v = __shfl_up_sync(0xffffffffu, inclusive, d);
          if (lane >= d) inclusive += v;
        }
        const uint32_t totals = __shfl_sync(0xffffffffu, inclusive, 31);
        const uint32_t t0 = totals & 0xffu, t1 = (totals >> 8) & 0xffu, t2 = (totals >> 16) & 0xffu;
        const uint32_t exclusive = inclusive - packed;
        const uint32_t base = kept + table[c * 32u + warp];
        const uint32_t all = mask;
        while (mask) {  // few scores pass: visit only those
          const uint32_t bit = __ffs(mask) - 1u, u = bit >> 2;
          mask &= mask - 1u;
          const uint32_t earlier = (u > 0u ? t0 : 0u) + (u > 1u ? t1 : 0u) + (u > 2u ? t2 : 0u);
          const uint32_t within = __popc(all & (0xfu << (4u * u)) & ((1u << bit) - 1u));
          const uint32_t slot = base + earlier + ((exclusive >> (8u * u)) & 0xffu) + within;
          if (slot < kPivotCandidates) list_pos[slot] = run + u * 128u + lane * 4u + (bit & 3u);
        }
      }
      kept += total;
      __syncthreads();  // the table is rewritten by the next round
    }
  }
  __syncthreads();
  if (ranks > 1u) {
    // hand the other slices' lists to rank 0 in rank order: positions stay in order
    if (tid == 0) kept_here = kept;
    cluster.sync();  // all lists and counts are complete
    if (rank == 0) {
      for (uint32_t r = 1; r < ranks; ++r) {
        const uint32_t theirs = *cluster.map_shared_rank(&kept_here, r);
        if (kept <= kPivotCandidates && theirs <= kPivotCandidates - kept) {
          const uint32_t* remote = cluster.map_shared_rank(list_pos, r);
          for (uint32_t i = tid; i < theirs; i += kThreads) list_pos[kept + i] = remote[i];
          kept += theirs;
        } else {
          kept = kPivotCandidates + 1u;  // does not fit: three passes over the row instead
        }
      }
    }
    cluster.sync();  // rank 0 has read the other CTAs' shared memory
    if (rank != 0) return;
    __syncthreads();
  }
  if (kept < kTop || kept > kPivotCandidates) {  // block-uniform: the sample misled, or the row is (nearly) constant
    select_row(a, row, nullptr);
    return;
  }

  for (uint32_t i = tid; i < kept; i += kThreads) list_key[i] = sortable_key(scores[list_pos[i]]);
  __syncthreads();

  // ---- 3. exact 2048th key among the kept ---------------------------------------------------------------
  // Three radix passes (12 + 12 + 8 bits) over the list. The histogram is cleared once; in every pass the thread
  // that scans a group of bins takes them into registers and clears them for the next pass, so a pass costs four
  // block barriers: after the adds, two inside the scan, and before the digit is read.
  uint32_t prefix = 0, prefix_mask = 0, remaining = kTop;
  for (uint32_t i = tid; i < 4096u; i += kThreads) hist[i] = 0;
  __syncthreads();
#pragma unroll 1
  for (uint32_t pass = 0; pass < 3; ++pass) {
    const uint32_t bits = pass == 2 ? 8u : 12u;
    const uint32_t shift = pass == 0 ? 20u : (pass == 1 ? 8u : 0u);
    const uint32_t bins = 1u << bits;
    for (uint32_t r = 0; r * kThreads < kept; ++r) {  // block-uniform trip count: hist_add votes per warp
      const uint32_t i = r * kThreads + tid;
      const uint32_t key = i < kept ? list_key[i] : 0u;
      hist_add(hist, i < kept && (key & prefix_mask) == prefix, (key >> shift) & (bins - 1u));
    }
    __syncthreads();
    const uint32_t per = bins / kThreads ? bins / kThreads : 1u;  // 4, 4, then 1 (256 bins)
    const uint32_t groups = bins / per;
    const uint32_t group = groups - 1u - tid;  // valid when tid < groups
    uint32_t count[4] = {0u, 0u, 0u, 0u}, local = 0;
    if (tid < groups) {
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j)
        if (j < per) {
          count[j] = hist[group * per + j];
          hist[group * per + j] = 0;   // nobody adds to it before the barrier that ends this pass
          local += count[j];
        }
    }
    uint32_t above = block_exclusive_scan(local, scan_scratch, nullptr);
    if (tid < groups) {
#pragma unroll
      for (int32_t j = 3; j >= 0; --j)
        if (static_cast<uint32_t>(j) < per) {
          if (above < remaining && above + count[j] >= remaining) {
            found[0] = group * per + static_cast<uint32_t>(j);
            found[1] = remaining - above;
          }
          above += count[j];
        }
    }
    __syncthreads();
    prefix |= found[0] << shift;   // rewritten only after the next pass's barriers
    prefix_mask |= (bins - 1u) << shift;
    remaining = found[1];
  }
  const uint32_t kth = prefix;         // exact key of the 2048th largest element
  const uint32_t need_eq = remaining;  // how many == kth positions are taken
  const uint32_t count_gt = kTop - need_eq;

  // ---- 4. emission: the list is in position order ---------------------------------------------------------
  const uint32_t groups = (kept + kThreads - 1u) / kThreads;  // groups of 32 list entries per warp
  const uint32_t run = warp * (32u * groups);
  uint32_t warp_gt = 0, warp_eq = 0;
  for (uint32_t j = 0; j < groups; ++j) {
    const uint32_t i = run + j * 32u + lane;
    const uint32_t key = i < kept ? list_key[i] : 0u;
    warp_gt += __popc(__ballot_sync(0xffffffffu, i < kept && key > kth));
    warp_eq += __popc(__ballot_sync(0xffffffffu, i < kept && key == kth));
  }
  uint32_t offset = block_exclusive_scan(lane == 0 ? (warp_gt | (warp_eq << 16)) : 0u, scan_scratch, nullptr);
  offset = __shfl_sync(0xffffffffu, offset, 0);
  uint32_t g = offset & 0xffffu, q = offset >> 16;
  for (uint32_t j = 0; j < groups; ++j) {
    const uint32_t i = run + j * 32u + lane;
    const uint32_t key = i < kept ? list_key[i] : 0u;
    const uint32_t mask_gt = __ballot_sync(0xffffffffu, i < kept && key > kth);
    const uint32_t mask_eq = __ballot_sync(0xffffffffu, i < kept && key == kth);
    uint32_t at = kTop;
    if ((mask_gt >> lane) & 1u) {
      at = g + __popc(mask_gt & below);
    } else if ((mask_eq >> lane) & 1u) {
      const uint32_t tie = q + __popc(mask_eq & below);
      if (tie < need_eq) at = count_gt + tie;
    }
    if (at < kTop) {
      const uint32_t position = list_pos[i];
      out[at] = static_cast<int32_t>(position + a.base_index);
      if (out_scores) out_scores[at] = scores[position];
    }
    g += __popc(mask_gt);
    q += __popc(mask_eq);
  }
}

}  // namespace

uint32_t launch_topk_pivot(const KvipTopkArgs& a, cudaStream_t stream) {
  constexpr int kSmem = static_cast<int>(2u * kPivotCandidates * sizeof(uint32_t));
  if (uint32_t bad = raise_dynamic_smem(kSlotTopkPivot, reinterpret_cast<const void*>(topk_pivot), kSmem,
                                        "topk_pivot attribute"))
    return bad;
  // two, four or eight CTAs per row while the clusters still fit the GPU in one wave (a cluster of eight
  // 1024-thread CTAs needs eight free SMs of one GPC: about two of them fit per GPC)
  const unsigned sms = device_sm_count();
  // (a cluster of eight pays for itself only on long rows: its barriers and the hand-over of eight lists cost more
  // than the shorter filter saves below about 256k scores - one row of 131072: 20.3 us on four CTAs, 22.6 on eight)
  const unsigned most = a.scoreStride >= 262144u ? 8u : 4u;
  const unsigned fit = 8u * a.rows <= (sms * 3u) / 4u ? 8u : (4u * a.rows <= (sms * 7u) / 8u ? 4u : (2u * a.rows <= sms ? 2u : 1u));
  const unsigned ranks = fit < most ? fit : most;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a.rows * ranks, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = kSmem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = ranks;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, topk_pivot, a) != cudaSuccess) return check_launch("topk_pivot");
  count_launch();
  return check_launch("topk_pivot");
}

}  // namespace kvip
