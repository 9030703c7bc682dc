// Lightning-indexer score on tcgen05 tensor cores.
//
//   score[t, s] = kscale[s] * sum_h W[t, h] * relu( q[t, h, :] . k[s, :] )
//
// What the reference computes in QLIMatmul::ComputeMm1 + ProcessVec1
// (op_kernel/indexer/indexer_cube.h:161-322, indexer_vector.h:513-662,
// indexer_score.h:59-140, 384-426), re-designed for sm_100a:
//
//   * the 128-token key page is the M operand (one TMA box per page of the paged Index
//     cache, 128-byte swizzle), the request's query heads are the N operand, so the
//     accumulator in tensor memory has one LANE per token and one COLUMN per
//     (query, head). The ReLU * W reduction over heads is then a per-thread loop over
//     columns: no cross-lane shuffle, no shared-memory transpose;
//   * persistent CTAs (one per SM) walk a flat list of (request, page) tiles, so a
//     request's keys and scales are streamed from HBM exactly once for all of its
//     query rows;
//   * warp 0 = TMA producer, warps 1-4 = MMA issuers that take tiles round-robin (warp 1 owns
//     tensor memory), warps 5-7 idle (they pad the control roles to two whole warpgroups), warps 8-23 = four
//     epilogue groups that take tiles round-robin; key
//     stages and a ring of up to eight accumulator buffers in tensor memory are handed over
//     with mbarriers. The number of issuers divides the number of key stages and of
//     accumulators, and the number of units reduced at once divides the number of accumulators, so
//     every use of one stage or accumulator is waited for by the same thread, in order: a
//     parity wait by a thread that runs a whole phase ahead of the barrier would pass at once;
//   * every mbarrier wait is bounded: when a wait gives up the CTA sets
//     KVIP_ERR_PIPELINE in the status word, all roles leave their loops, tensor memory
//     is released and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "common.cuh"

namespace kvip {
namespace {

constexpr uint32_t kEpilogueGroups = 4;
constexpr uint32_t kMmaWarps = 4;          // MMA issuers: warps 1..4 (one thread each)
// Warps 0-7 are two "control" warpgroups (producer, four issuers, three idle warps), warps 8-23 four epilogue
// warpgroups: register budgets are moved between whole warpgroups (setmaxnreg), from the control warps, which need
// few, to the epilogue warps, which keep 64 accumulator columns in registers at a time.
constexpr uint32_t kFirstEpilogueWarp = 8; // any four consecutive warps cover the four tensor-memory lane quadrants
constexpr uint32_t kControlRegisters = 48, kEpilogueRegisters = 96;
constexpr uint32_t kLiThreads = 32 * kFirstEpilogueWarp + 128 * kEpilogueGroups;
constexpr uint32_t kMaxAcc = 8;       // accumulator buffers in tensor memory (512 columns / stride)
constexpr uint32_t kMaxBatch = 1024;
constexpr uint32_t kMaxN = 256;            // query slots * heads
constexpr uint32_t kAtomBytes = 128 * 128; // one 128-row x 128-byte swizzle atom
constexpr uint32_t kDefaultWaitKilocycles = 2000000u;  // about one second of SM clock

template <bool kBf16> struct LiCfg {
  static constexpr uint32_t kAtoms = kBf16 ? 2 : 1;           // 128-byte K slices per row
  static constexpr uint32_t kTileBytes = kAtomBytes * kAtoms; // one key page in smem
  static constexpr uint32_t kMaxStages = 8;   // more than eight 16 KB stages in flight per SM measured slower
  static constexpr uint32_t kSmemLimit = 227 * 1024;
  // everything but the key stages, for `n` = query slots x heads accumulator columns
  static constexpr uint32_t fixed_bytes(uint32_t n) {
    return 1024 /*alignment slack*/ + 1024 /*barriers*/ + n * 128 * kAtoms /*query tile*/ +
           4 * kEpilogueGroups * n * 4 /*W per epilogue warp*/ + (kMaxBatch + 1) * 4 /*tile prefix*/ +
           kMaxBatch /*active queries*/ + 64;
  }
  // as many key stages as shared memory holds: bytes in flight are what saturates HBM
  static constexpr uint32_t stages_for(uint32_t n) {
    const uint32_t s = (kSmemLimit - fixed_bytes(n)) / kTileBytes;
    return s > kMaxStages ? kMaxStages : s;
  }
};

// ---- PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait. Returns false when the CTA is aborting (this wait or another one gave up).
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0u;
}
// Up to 64 tries in one tight loop (four instructions per try): waiting threads share their schedulers with the
// epilogue warps, so every instruction a wait loop issues is taken from them.
__device__ __forceinline__ bool mbar_try_64(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .u32 n;\n\t"
      "mov.u32 n, 64;\n\t"
      "TRY_AGAIN:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra TRY_DONE;\n\t"
      "sub.u32 n, n, 1;\n\t"
      "setp.ne.u32 q, n, 0;\n\t"
      "@q bra TRY_AGAIN;\n\t"
      "TRY_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0u;
}
struct WaitControl {
  volatile uint32_t* abort_flag;   // set by the first wait of the CTA that gives up; read by all the others
  long long limit;                 // SM clock cycles a wait may take
};
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitControl& control) {
  if (mbar_try(bar, parity)) return true;  // the common case costs one instruction
  const long long start = clock64();
  for (;;) {
    if (mbar_try_64(bar, parity)) return true;
    if (*control.abort_flag) return false;
    if (clock64() - start > control.limit) break;
  }
  *control.abort_flag = 1u;
  return false;
}
// Two fp32 fused multiply-adds in one instruction (packed pairs in 64-bit registers): the epilogue is bound by
// the instructions it issues per accumulator column, and this halves the fma count. Each lane rounds like fmaf.
__device__ __forceinline__ uint64_t pack_f32x2(float low, float high) {
  uint64_t packed;
  asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "f"(low), "f"(high));
  return packed;
}
__device__ __forceinline__ void fma_f32x2(uint64_t& acc, uint64_t x, uint64_t w) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(x), "l"(w));
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
template <bool kBf16>
__device__ __forceinline__ void tcgen05_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  if constexpr (kBf16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 32 columns of fp32: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

struct TileCursor {  // walks the flat (request, page) list shared by the three roles
  const uint32_t* prefix;
  uint32_t batch, request, limit;   // limit: first tile of the next request (kept in a register: the common call
                                    // is one compare, not a shared-memory round trip)
  __device__ TileCursor(const uint32_t* p, uint32_t b) : prefix(p), batch(b), request(0), limit(b > 1u ? p[1] : 0xffffffffu) {}
  __device__ uint32_t seek(uint32_t tile) {
    while (tile >= limit) {
      ++request;
      limit = request + 1 < batch ? prefix[request + 1] : 0xffffffffu;
    }
    return request;
  }
};

__device__ __forceinline__ float load_weight(const KvipLiArgs& a, uint32_t index) {
  float w;
  if (a.weightDtype == KVIP_WEIGHT_FP32) {
    w = reinterpret_cast<const float*>(a.weights)[index];
  } else {
    w = __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(a.weights)[index]) << 16);
  }
  if (a.query_scale) w *= a.query_scale[index];
  return w;
}

template <bool kBf16>
__global__ void __launch_bounds__(kLiThreads, 1)
li_score_tcgen05(const __grid_constant__ CUtensorMap key_map, const __grid_constant__ CUtensorMap query_map,
                 const __grid_constant__ KvipLiArgs a, const uint32_t S) {
  using Cfg = LiCfg<kBf16>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  // layout from the 1024-byte aligned base: [barriers + control, 1024 B][key stages][query tile]
  // [W per epilogue warp][tile prefix][active queries]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  const uint32_t key_smem = base + 1024u;
  const uint32_t n_max = a.queries * a.heads;  // accumulator columns / query-tile rows of this launch
  const uint32_t q_atom_bytes = n_max * 128u;  // one 128-byte K slice of the query tile
  const uint32_t q_smem = key_smem + S * Cfg::kTileBytes;
  float* w_smem = reinterpret_cast<float*>(smem + 1024u + S * Cfg::kTileBytes + q_atom_bytes * Cfg::kAtoms);
  uint32_t* prefix = reinterpret_cast<uint32_t*>(w_smem + 4 * kEpilogueGroups * n_max);
  uint8_t* active_q = reinterpret_cast<uint8_t*>(prefix + kMaxBatch + 1);
  // barrier map: [0,S) full, [S,2S) empty, 2S q_full, 2S+1 q_empty, then kMaxAcc tmem_full and kMaxAcc
  // tmem_empty; then the tmem base word and the abort flag.
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](uint32_t i) { return bar0 + i * 8u; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 2 + 2 * kMaxAcc);
  const uint32_t kQFull = 2 * S, kQEmpty = 2 * S + 1, kAccFull = 2 * S + 2, kAccEmpty = 2 * S + 2 + kMaxAcc;
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const WaitControl waits{abort_flag, static_cast<long long>(a.wait_kilocycles ? a.wait_kilocycles : kDefaultWaitKilocycles) << 10};

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t H = a.heads, Q = a.queries, pages = a.pagesPerRequest;
  // A tile (key page x query rows of the request) is handed over in UNITS of at most 128 accumulator columns:
  // one unit per tile up to 128 (query, head) columns, two beyond (queries 0-1 and 2-3 at 64 heads). Four units
  // fit tensor memory at 128 columns each, so MMA and reduction overlap even for the widest query tile.
  const uint32_t halves = Q * H > 128u ? 2u : 1u;
  const uint32_t halves_shift = halves - 1u;   // halves is 1 or 2: unit -> tile is a shift, not a division (a 32-bit
                                               // division by a run-time value costs about a hundred cycles, and the
                                               // epilogue did four per unit)
  const uint32_t unit_queries = halves == 2u ? 128u / H : Q;    // query slots per unit
  const uint32_t acc_stride = Q * H <= 32u ? 32u : (Q * H <= 64u ? 64u : 128u);
  const uint32_t acc_count = min(kMaxAcc, 512u / acc_stride);   // 4 or 8
  // issuer w owns the units of the tiles with local index = w (mod issuers): the accumulators of those units
  // must be the same every time round the ring, i.e. issuers * halves divides acc_count (and issuers divides S)
  const uint32_t acc_tiles = acc_count / halves;
  // Four issuers are needed where a key page arrives every ~370 ns (64 columns: the kernel is memory-bound); from 128
  // columns on the epilogue sets the pace, two issuers keep up with it, and two fewer waiting warps leave their issue
  // slots to the epilogue warps of the same schedulers (measured: 52.0 against 53.9 us; one issuer: 64.5).
  const uint32_t issuers_most = Q * H >= 128u ? 2u : 4u;
  const uint32_t issuers = min(issuers_most, ((S | acc_tiles) & 3u) == 0u ? 4u : (((S | acc_tiles) & 1u) == 0u ? 2u : 1u));
  const uint32_t groups = kEpilogueGroups;   // units reduced concurrently; divides acc_count (4 or 8)

  // ---- per-CTA schedule: tiles per request -> prefix sums (warp 0) -------------------
  if (warp == 0) {
    uint32_t carry = 0;
    if (lane == 0) prefix[0] = 0;
    for (uint32_t b0 = 0; b0 < a.batch; b0 += 32) {
      const uint32_t b = b0 + lane;
      uint32_t tiles = 0, nq = 0;
      if (b < a.batch) {
        int32_t longest = 0;
        for (uint32_t q = 0; q < Q; ++q) {
          const int32_t end = a.query_ends[b * Q + q];
          if (end > 0) { nq = q + 1; longest = max(longest, end); }
        }
        int32_t len = min(a.key_lengths[b], longest);
        len = min(len, static_cast<int32_t>(pages * kBlockTokens));
        if (nq && len > 0) tiles = (static_cast<uint32_t>(len) + kBlockTokens - 1) / kBlockTokens;
        active_q[b] = static_cast<uint8_t>(tiles ? nq : 0);
      }
      uint32_t scan = tiles;
#pragma unroll
      for (uint32_t d = 1; d < 32; d <<= 1) {
        uint32_t v = __shfl_up_sync(0xffffffffu, scan, d);
        if (lane >= d) scan += v;
      }
      if (b < a.batch) prefix[b + 1] = carry + scan;
      carry += __shfl_sync(0xffffffffu, scan, 31);
    }
  }
  if (threadIdx.x == 64) {
    for (uint32_t i = 0; i < S; ++i) { mbar_init(bar(i), 1); mbar_init(bar(S + i), 1); }
    mbar_init(bar(kQFull), 1); mbar_init(bar(kQEmpty), issuers);
    for (uint32_t i = 0; i < kMaxAcc; ++i) { mbar_init(bar(kAccFull + i), 1); mbar_init(bar(kAccEmpty + i), 128u); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory: all 512 columns (one CTA per SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
                     smem_u32(const_cast<uint32_t*>(tmem_slot)))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t total_tiles = prefix[a.batch];
  const uint32_t tile_begin = static_cast<uint32_t>((static_cast<uint64_t>(total_tiles) * blockIdx.x) / gridDim.x);
  const uint32_t tile_end = static_cast<uint32_t>((static_cast<uint64_t>(total_tiles) * (blockIdx.x + 1)) / gridDim.x);

  // 768 threads start with 80 registers each; the control warpgroups give 2 x 128 x 32 back and the epilogue
  // warpgroups take 4 x 128 x 16 of them
  if (warp < kFirstEpilogueWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegisters));
  if (warp == 0) {
    // ================= TMA producer =================
    // The whole warp stays in the loop: each lane looks up the page of one of the next 32 tiles (one
    // coalesced read of the block table, issued a full group ahead), lane 0 issues the copies. A page
    // lookup is a dependent global load; done per tile by the issuing thread it would serialise the
    // pipeline on memory latency.
    TileCursor lane_cursor(prefix, a.batch);
    auto lookup = [&](uint32_t t, uint32_t* request) -> int32_t {
      if (t >= tile_end) { *request = 0; return 0; }
      const uint32_t b = lane_cursor.seek(t);
      *request = b;
      return a.block_table[static_cast<uint64_t>(b) * pages + (t - prefix[b])];
    };
    uint32_t stage = 0, phase = 0, loaded_q = 0, alive = 1;
    int32_t bound = -1;
    uint32_t next_request;
    int32_t next_page = lookup(tile_begin + lane, &next_request);
    for (uint32_t base = tile_begin; base < tile_end && alive; base += 32) {
      const int32_t my_page = next_page;
      const uint32_t my_request = next_request;
      next_page = lookup(base + 32 + lane, &next_request);   // lands while this group is being issued
      const uint32_t count = min(32u, tile_end - base);
      for (uint32_t i = 0; i < count && alive; ++i) {
        const int32_t page = __shfl_sync(0xffffffffu, my_page, i);
        const uint32_t b = __shfl_sync(0xffffffffu, my_request, i);
        if (lane == 0) {
          if (static_cast<int32_t>(b) != bound) {
            if (mbar_wait(bar(kQEmpty), (loaded_q & 1u) ^ 1u, waits)) {
              const uint32_t rows = active_q[b] * H;
              mbar_expect_tx(bar(kQFull), rows * 128u * Cfg::kAtoms);
              for (uint32_t atom = 0; atom < Cfg::kAtoms; ++atom)
                for (uint32_t r = 0; r < rows; r += 32)
                  tma_load_2d(q_smem + atom * q_atom_bytes + r * 128u, &query_map,
                              static_cast<int32_t>(atom * 64u), static_cast<int32_t>(b * Q * H + r),
                              bar(kQFull));
              ++loaded_q;
              bound = static_cast<int32_t>(b);
            } else {
              alive = 0;
            }
          }
          if (alive && mbar_wait(bar(S + stage), phase ^ 1u, waits)) {
            // test hook: the withheld page never arrives, its consumer's bounded wait gives up
            const bool withheld = a.withhold_tile && blockIdx.x == 0 && base + i - tile_begin + 1u == a.withhold_tile;
            if (!withheld) {
              mbar_expect_tx(bar(stage), Cfg::kTileBytes);
              for (uint32_t atom = 0; atom < Cfg::kAtoms; ++atom)
                tma_load_2d(key_smem + stage * Cfg::kTileBytes + atom * kAtomBytes, &key_map,
                            static_cast<int32_t>(atom * 64u), page * static_cast<int32_t>(kBlockTokens), bar(stage));
            }
            if (++stage == S) { stage = 0; phase ^= 1u; }
          } else {
            alive = 0;
          }
        }
        alive = __shfl_sync(0xffffffffu, alive, 0);
      }
    }
  } else if (warp <= kMmaWarps) {
    // ================= MMA issuers =================
    // Issuer w (one thread of warp 1 + w) takes the tiles with (t - tile_begin) % issuers == w. Issuing
    // a tcgen05 instruction occupies the issuing thread for tens of nanoseconds, and a page needs four MMAs
    // and two commits: one thread alone caps the SM below the rate at which key pages arrive from HBM.
    // Tiles are independent (each has its own accumulator), so the issuers need no order among themselves.
    // The query operand is shared: every issuer waits for each request's query tile and arrives on the
    // q_empty barrier once per request, by tcgen05.commit if it issued MMAs that read the tile.
    const uint32_t w = warp - 1u;
    if (lane == 0 && w < issuers && tile_begin < tile_end) {
      TileCursor cur(prefix, a.batch);
      uint32_t request = cur.seek(tile_begin), seq = 0;
      uint32_t t = tile_begin + w;
      uint32_t stage = w, phase = 0;                           // w < issuers <= S
      uint32_t acc = w * halves, acc_phase = 0;                // first unit of tile w; w * halves < acc_count
      bool alive = true;
      while (alive) {
        const uint32_t request_end = min(prefix[request + 1], tile_end);
        if (!mbar_wait(bar(kQFull), seq & 1u, waits)) break;
        const uint32_t n = active_q[request] * H;              // live accumulator columns of this request
        const uint32_t fmt = kBf16 ? 1u : 0u;  // kind::f16: BF16 = 1; kind::f8f6f4: E4M3 = 0
        bool issued = false;
        for (; t < request_end; t += issuers) {
          if (!mbar_wait(bar(stage), phase, waits)) { alive = false; break; }
          for (uint32_t h = 0; h < halves; ++h) {
            if (!mbar_wait(bar(kAccEmpty + acc + h), acc_phase ^ 1u, waits)) { alive = false; break; }
            const uint32_t first_column = h * 128u;
            if (n <= first_column) {                 // no live query slot in this unit: nothing to compute
              mbar_arrive(bar(kAccFull + acc + h));
              continue;
            }
            const uint32_t columns = min(n - first_column, halves == 2u ? 128u : n);
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((columns >> 3) << 17) | ((128u >> 4) << 24);
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem_base + (acc + h) * acc_stride;
#pragma unroll
            for (uint32_t atom = 0; atom < Cfg::kAtoms; ++atom) {
              const uint64_t da = umma_desc(key_smem + stage * Cfg::kTileBytes + atom * kAtomBytes);
              const uint64_t db = umma_desc(q_smem + atom * q_atom_bytes + first_column * 128u);
#pragma unroll
              for (uint32_t k = 0; k < 4; ++k)  // 32 bytes of K per instruction
                tcgen05_mma<kBf16>(d_tmem, da + 2u * k, db + 2u * k, idesc, (atom | k) != 0u);
            }
            tcgen05_commit(bar(kAccFull + acc + h));   // accumulator ready for the epilogue
          }
          if (!alive) break;
          tcgen05_commit(bar(S + stage));              // key stage free once these MMAs retire
          issued = true;
          stage += issuers;
          if (stage >= S) { stage -= S; phase ^= 1u; }
          acc += issuers * halves;
          if (acc >= acc_count) { acc -= acc_count; acc_phase ^= 1u; }
        }
        if (!alive) break;
        if (issued) tcgen05_commit(bar(kQEmpty));  // query operand may be replaced once my MMAs retire
        else mbar_arrive(bar(kQEmpty));
        if (request_end >= tile_end) break;
        do { ++request; } while (prefix[request + 1] == prefix[request]);  // next request that has tiles
        ++seq;
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegisters));
    // ================= epilogue: groups of 4 warps, one token row per thread =================
    // One unit's reduction is a long dependent chain (tensor-memory load, 64 max+fma pairs per query, store),
    // far longer than the time the next key page needs to arrive, so several units are reduced concurrently.
    const uint32_t group = (warp - kFirstEpilogueWarp) >> 2;
    const uint32_t quad = warp & 3u;              // tensor-memory lane quadrant of this warp
    const uint32_t row = quad * 32u + lane;       // token row inside the page
    float* w_warp = w_smem + (warp - kFirstEpilogueWarp) * n_max;  // private copy: no cross-warp barrier needed
    TileCursor cur(prefix, a.batch), ahead(prefix, a.batch);
    uint32_t live_mask = 0;
    int32_t bound = -1;
    // The page index and the key scale of a tile are two dependent global loads. They are issued two
    // and one of this group's tiles ahead, so their latency is hidden behind the tile being reduced.
    auto page_of = [&](uint32_t t) -> int32_t {
      if (t >= tile_end) return 0;
      const uint32_t b = ahead.seek(t);
      return a.block_table[static_cast<uint64_t>(b) * pages + (t - prefix[b])];
    };
    auto scale_of = [&](uint32_t t, int32_t page) -> float {
      if (t >= tile_end || !a.key_scale) return 1.0f;
      return a.key_scale[static_cast<uint64_t>(page) * kBlockTokens + row];
    };
    // Group g reduces the units u = g (mod groups); unit u is half (u mod halves) of tile u / halves.
    const uint32_t G = groups;
    const uint32_t tiles_here = tile_end - tile_begin, units_here = tiles_here * halves;
    auto tile_of = [&](uint32_t u) { return u < units_here ? tile_begin + (u >> halves_shift) : tile_end; };
    const uint32_t first = group;
    int32_t page_next = page_of(tile_of(first));
    float kscale = scale_of(tile_of(first), page_next);
    page_next = page_of(tile_of(first + G));
    uint32_t acc = group % acc_count, acc_phase = 0;   // G divides acc_count: a group meets the same accumulators
    for (uint32_t u = first; u < units_here; u += G) {
      const uint32_t t = tile_begin + (u >> halves_shift), h = u & (halves - 1u);
      const uint32_t b = cur.seek(t);
      const uint32_t nq = active_q[b];
      const float kscale_next = scale_of(tile_of(u + G), page_next);   // consumed next iteration
      page_next = page_of(tile_of(u + 2 * G));
      if (static_cast<int32_t>(b) != bound) {
        __syncwarp();
        for (uint32_t i = lane; i < nq * H; i += 32u) w_warp[i] = load_weight(a, b * Q * H + i);
        live_mask = 0;
        for (uint32_t q = 0; q < nq; ++q) live_mask |= (a.query_ends[b * Q + q] > 0 ? 1u : 0u) << q;
        __syncwarp();
        bound = static_cast<int32_t>(b);
      }
      const uint32_t token = (t - prefix[b]) * kBlockTokens + row;
      // warp-uniform outcome: the tensor-memory loads below need the whole warp
      if (!__all_sync(0xffffffffu, mbar_wait(bar(kAccFull + acc), acc_phase, waits))) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + acc * acc_stride;
      const uint32_t q_first = h * unit_queries, q_last = min(nq, q_first + unit_queries);
      for (uint32_t q = q_first; q < q_last; ++q) {
        // four independent accumulation chains (heads 0,4,8.. / 1,5,.. / 2,6,.. / 3,7,..): the sum over heads
        // is compared with a tolerance, so its order is free, and the chains give the FMA pipe work to overlap
        uint64_t s01 = 0ull, s23 = 0ull;   // (s0, s1) and (s2, s3) as packed pairs
        auto reduce = [&](const uint32_t(&v)[32], uint32_t c) {
          const ulonglong2* w4 = reinterpret_cast<const ulonglong2*>(w_warp + q * H + c);
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            const ulonglong2 w = w4[j];   // (w0, w1), (w2, w3)
            fma_f32x2(s01, pack_f32x2(fmaxf(__uint_as_float(v[4 * j + 0]), 0.f), fmaxf(__uint_as_float(v[4 * j + 1]), 0.f)), w.x);
            fma_f32x2(s23, pack_f32x2(fmaxf(__uint_as_float(v[4 * j + 2]), 0.f), fmaxf(__uint_as_float(v[4 * j + 3]), 0.f)), w.y);
          }
        };
        if (H == 64u) {
          // both halves of the slot's columns behind ONE wait: alone a tensor-memory load comes back in tens of
          // cycles, but here it queues behind the MMAs in flight and takes hundreds, and a warp has nothing else
          // to do meanwhile
          uint32_t lower[32], upper[32];
          tmem_ld_32x32(taddr + (q - q_first) * 64u, lower);
          tmem_ld_32x32(taddr + (q - q_first) * 64u + 32u, upper);
          tmem_ld_wait();
          reduce(lower, 0u);
          reduce(upper, 32u);
        } else {
          uint32_t v[32];
          tmem_ld_32x32(taddr + (q - q_first) * 32u, v);
          tmem_ld_wait();
          reduce(v, 0u);
        }
        if ((live_mask >> q) & 1u) {
          const float s0 = __uint_as_float(static_cast<uint32_t>(s01)), s1 = __uint_as_float(static_cast<uint32_t>(s01 >> 32));
          const float s2 = __uint_as_float(static_cast<uint32_t>(s23)), s3 = __uint_as_float(static_cast<uint32_t>(s23 >> 32));
          float score = ((s0 + s2) + (s1 + s3)) * kscale;   // (even heads) + (odd heads)
          if (a.scoreMode == KVIP_SCORE_BF16_AWAY) score = bf16_away(score);
          a.scores[static_cast<uint64_t>(b * Q + q) * a.scoreStride + token] = score;
        }
      }
      tcgen05_fence_before();
      mbar_arrive(bar(kAccEmpty + acc));
      acc += G;
      if (acc >= acc_count) { acc -= acc_count; acc_phase ^= 1u; }
      kscale = kscale_next;
    }
  }

  // ---- teardown ------------------------------------------------------------------------
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(a.status, static_cast<int32_t>(KVIP_ERR_PIPELINE));
    // give copies and MMAs that may still be in flight time to land before the CTA's
    // shared and tensor memory are released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---- CUDA-core cross-check ------------------------------------------------------------
// One thread per (query row, token). Products are accumulated over d = 0..127 with fmaf in
// ascending order, heads with the even/odd fmaf chains of indexer_score.h:59-140: the same
// arithmetic, in the same order, as the CPU oracle.
__device__ __forceinline__ float decode_e4m3(uint8_t code) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(code), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__global__ void __launch_bounds__(128) li_score_simt(const KvipLiArgs a) {
  extern __shared__ float q_f32[];  // [heads * 128]
  const uint32_t t = blockIdx.y, b = t / a.queries;
  const int32_t end = a.query_ends[t];
  const int32_t len = min(min(a.key_lengths[b], end), static_cast<int32_t>(a.pagesPerRequest * kBlockTokens));
  const uint32_t token = blockIdx.x * 128u + threadIdx.x;
  if (end <= 0 || static_cast<int32_t>(blockIdx.x * 128u) >= len) return;
  const uint32_t H = a.heads;
  for (uint32_t i = threadIdx.x; i < H * 128u; i += 128u) {
    const uint64_t src = static_cast<uint64_t>(t) * H * 128u + i;
    q_f32[i] = a.keyDtype == KVIP_KEY_BF16
                   ? __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(a.query)[src]) << 16)
                   : decode_e4m3(reinterpret_cast<const uint8_t*>(a.query)[src]);
  }
  __syncthreads();
  const int32_t page = a.block_table[static_cast<uint64_t>(b) * a.pagesPerRequest + blockIdx.x];
  const uint64_t key_row = static_cast<uint64_t>(page) * kBlockTokens + threadIdx.x;
  float even = 0.f, odd = 0.f;
  for (uint32_t h = 0; h < H; ++h) {
    float dot = 0.f;
    for (uint32_t d = 0; d < 128u; ++d) {
      const float k = a.keyDtype == KVIP_KEY_BF16
                          ? __uint_as_float(static_cast<uint32_t>(
                                reinterpret_cast<const uint16_t*>(a.keys)[key_row * 128u + d]) << 16)
                          : decode_e4m3(reinterpret_cast<const uint8_t*>(a.keys)[key_row * 128u + d]);
      dot = fmaf(q_f32[h * 128u + d], k, dot);
    }
    const float w = load_weight(a, t * H + h);
    if (h & 1u) odd = fmaf(fmaxf(dot, 0.f), w, odd);
    else even = fmaf(fmaxf(dot, 0.f), w, even);
  }
  float score = (even + odd) * (a.key_scale ? a.key_scale[key_row] : 1.0f);
  if (a.scoreMode == KVIP_SCORE_BF16_AWAY) score = bf16_away(score);
  a.scores[static_cast<uint64_t>(t) * a.scoreStride + token] = score;
}

// ---- host side -------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &qres) !=
            cudaSuccess || qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

bool encode_rows_map(CUtensorMap* map, const void* base, uint64_t rows, bool bf16, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {128, rows};
  const cuuint64_t strides[1] = {bf16 ? 256u : 128u};
  const cuuint32_t box[2] = {bf16 ? 64u : 128u, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
            const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

uint32_t validate(const KvipLiArgs* a) {
  KVIP_REQUIRE(a, "li_score: null argument struct");
  KVIP_REQUIRE(a->query && a->keys && a->weights && a->key_lengths && a->query_ends && a->block_table &&
                   a->scores && a->status, "li_score: null tensor pointer");
  KVIP_REQUIRE(a->batch >= 1 && a->batch <= kMaxBatch, "li_score: batch must be in 1..1024");
  KVIP_REQUIRE(a->queries >= 1 && a->queries <= KVIP_MAX_QUERIES, "li_score: 1..4 query slots per request");
  KVIP_REQUIRE(a->heads == 32 || a->heads == 64, "li_score: 32 or 64 index heads");
  KVIP_REQUIRE(a->pagesPerRequest >= 1 && a->scoreStride >= a->pagesPerRequest * kBlockTokens,
               "li_score: score rows must cover every page");
  KVIP_REQUIRE(a->keyRows >= kBlockTokens && a->keyRows % kBlockTokens == 0, "li_score: key rows must be whole pages");
  KVIP_REQUIRE(a->keyDtype <= KVIP_KEY_BF16 && a->weightDtype <= KVIP_WEIGHT_FP32 && a->scoreMode <= KVIP_SCORE_BF16_AWAY,
               "li_score: unknown dtype or score mode");
  KVIP_REQUIRE((reinterpret_cast<uintptr_t>(a->keys) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a->query) & 15u) == 0,
               "li_score: keys and query must be 16-byte aligned");
  return 0;
}

template <bool kBf16>
uint32_t launch_tcgen05(const KvipLiArgs& a, cudaStream_t stream) {
  using Cfg = LiCfg<kBf16>;
  CUtensorMap key_map, query_map;
  if (!encode_rows_map(&key_map, a.keys, a.keyRows, kBf16, 128) ||
      !encode_rows_map(&query_map, a.query, static_cast<uint64_t>(a.batch) * a.queries * a.heads, kBf16, 32)) {
    set_error("li_score: cuTensorMapEncodeTiled failed");
    return KVIP_BAD_ARGUMENT;
  }
  if (uint32_t bad = raise_dynamic_smem(kBf16 ? kSlotLiBf16 : kSlotLiFp8,
                                        reinterpret_cast<const void*>(li_score_tcgen05<kBf16>),
                                        static_cast<int>(Cfg::kSmemLimit), "li_score attribute"))
    return bad;
  const uint32_t n_max = a.queries * a.heads;
  uint32_t stages = Cfg::stages_for(n_max);
  if (a.stages && a.stages >= 2 && a.stages < stages) stages = a.stages;  // tuning knob: fewer key stages
  const uint32_t smem_bytes = Cfg::fixed_bytes(n_max) + stages * Cfg::kTileBytes;
  uint32_t ctas = a.ctas;
  if (!ctas) ctas = device_sm_count();
  li_score_tcgen05<kBf16><<<ctas, kLiThreads, smem_bytes, stream>>>(key_map, query_map, a, stages);
  count_launch();
  return check_launch("li_score_tcgen05");
}

}  // namespace

uint32_t launch_li_score(const KvipLiArgs& a, cudaStream_t stream) {
  return a.keyDtype == KVIP_KEY_BF16 ? launch_tcgen05<true>(a, stream) : launch_tcgen05<false>(a, stream);
}

uint32_t launch_li_score_simt(const KvipLiArgs& a, cudaStream_t stream) {
  dim3 grid(a.pagesPerRequest, a.batch * a.queries);
  li_score_simt<<<grid, 128, a.heads * 128 * sizeof(float), stream>>>(a);
  count_launch();
  return check_launch("li_score_simt");
}

}  // namespace kvip

extern "C" uint32_t kvip_b200_li_score(const KvipLiArgs* args, void* stream) {
  if (uint32_t bad = kvip::validate(args)) return bad;
  return kvip::launch_li_score(*args, static_cast<cudaStream_t>(stream));
}

extern "C" uint32_t kvip_b200_li_score_simt(const KvipLiArgs* args, void* stream) {
  if (uint32_t bad = kvip::validate(args)) return bad;
  return kvip::launch_li_score_simt(*args, static_cast<cudaStream_t>(stream));
}
