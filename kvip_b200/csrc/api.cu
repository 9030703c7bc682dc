// Host entry points of libkvip_b200.so: geometry, the fused forward and bookkeeping.
#include <atomic>
#include <cstdio>
#include <cstring>
#include "common.cuh"

namespace kvip {

uint32_t launch_li_score(const KvipLiArgs& a, cudaStream_t stream);
uint32_t launch_li_score_simt(const KvipLiArgs& a, cudaStream_t stream);
uint32_t launch_topk(const KvipTopkArgs& a, cudaStream_t stream);

uint32_t launch_resolve_requests(const KvipResolveArgs& a, cudaStream_t stream);
uint32_t launch_publish_outputs(const KvipResolveArgs& a, cudaStream_t stream);
uint32_t launch_exchange(const KvipExchangeArgs& a, cudaStream_t stream);
uint32_t launch_fetch(const KvipFetchArgs& a, cudaStream_t stream);
uint32_t launch_fetch_staged(const KvipFetchArgs& a, const KvipWorkspace& ws, cudaStream_t stream);
uint32_t launch_gather(const KvipGatherArgs& a, cudaStream_t stream);
uint32_t launch_publish_residency(const KvipFetchArgs& a, cudaStream_t stream);

namespace {
std::atomic<uint32_t> g_launches{0};
thread_local char g_error[256] = "";
}  // namespace

void count_launch(uint32_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void set_error(const char* message) {
  std::snprintf(g_error, sizeof(g_error), "%s", message);
}

uint32_t check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return 0;
  std::snprintf(g_error, sizeof(g_error), "%s: %s", what, cudaGetErrorString(e));
  return KVIP_CUDA_ERROR_BASE + static_cast<uint32_t>(e);
}

namespace {
constexpr int kMaxDevices = 64;
struct DeviceRecord {
  std::atomic<uint32_t> configured{0};   // bit per KernelSlot
  std::atomic<uint32_t> sm_count{0};
};
DeviceRecord g_devices[kMaxDevices];

DeviceRecord* current_device_record() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  return &g_devices[device];
}
}  // namespace

uint32_t raise_dynamic_smem(KernelSlot slot, const void* kernel, int bytes, const char* what) {
  DeviceRecord* record = current_device_record();
  const uint32_t bit = 1u << slot;
  if (record && (record->configured.load(std::memory_order_acquire) & bit)) return 0;
  // setting the attribute twice is harmless, so two threads racing here need no lock
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return check_launch(what);
  if (record) record->configured.fetch_or(bit, std::memory_order_release);
  return 0;
}

uint32_t device_sm_count() {
  DeviceRecord* record = current_device_record();
  if (record) {
    const uint32_t known = record->sm_count.load(std::memory_order_relaxed);
    if (known) return known;
  }
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return 148u;
  }
  if (record) record->sm_count.store(static_cast<uint32_t>(sms), std::memory_order_relaxed);
  return static_cast<uint32_t>(sms);
}

template <typename T> T* ptr(uint64_t word) { return reinterpret_cast<T*>(static_cast<uintptr_t>(word)); }

}  // namespace kvip

extern "C" uint32_t kvip_prepare_shape(KvipRuntimeShape* s) {
  using namespace kvip;
  KVIP_REQUIRE(s, "prepare_shape: null shape");
  KVIP_REQUIRE(s->batch >= 1 && s->batch <= 1024, "prepare_shape: batch must be in 1..1024");
  KVIP_REQUIRE(s->indexHeads == 32 || s->indexHeads == 64, "prepare_shape: 32 or 64 index heads");
  KVIP_REQUIRE(s->queries >= 1 && s->queries <= KVIP_MAX_QUERIES, "prepare_shape: 1..4 query slots per request");
  KVIP_REQUIRE(s->history % 128 == 0 && s->resident % 128 == 0, "prepare_shape: history/resident must align to 128");
  KVIP_REQUIRE(s->resident >= KVIP_TOPK && s->resident <= 131072, "prepare_shape: resident must be in 2048..131072");
  KVIP_REQUIRE(s->history >= s->resident && s->history <= (1u << 21), "prepare_shape: history must be in resident..2^21");
  KVIP_REQUIRE(s->tokenBytes >= 16 && s->tokenBytes % 16 == 0, "prepare_shape: token bytes must be a multiple of 16");
  KVIP_REQUIRE(s->keyDtype <= KVIP_KEY_BF16 && s->weightDtype <= KVIP_WEIGHT_FP32 && s->scoreMode <= KVIP_SCORE_BF16_AWAY &&
                   s->liVariant <= 1, "prepare_shape: unknown dtype, score mode or LI variant");
  s->pagesPerRequest = s->history / 128;
  s->scoreStride = s->history;
  s->finalWorkers = 4;
  if (!s->outputStride) s->outputStride = s->resident;
  KVIP_REQUIRE(s->outputStride >= s->resident, "prepare_shape: output stride must cover the resident slots");
  if (!s->owners) s->owners = s->batch;
  KVIP_REQUIRE(static_cast<uint64_t>(s->owners) * s->history <= 0xffffffffull, "prepare_shape: key rows overflow");
  if (!s->keyRows) s->keyRows = s->owners * s->history;
  return 0;
}

extern "C" uint32_t kvip_b200_host_register(void* host, uint64_t bytes, uint64_t* device_alias) {
  using namespace kvip;
  KVIP_REQUIRE(host && bytes && device_alias, "host_register: null argument");
  cudaError_t e = cudaHostRegister(host, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable);
  if (e != cudaSuccess) return check_launch("cudaHostRegister");
  void* alias = nullptr;
  e = cudaHostGetDevicePointer(&alias, host, 0);
  if (e != cudaSuccess) {
    cudaHostUnregister(host);
    return check_launch("cudaHostGetDevicePointer");
  }
  *device_alias = reinterpret_cast<uint64_t>(alias);
  return 0;
}

extern "C" uint32_t kvip_b200_host_unregister(void* host) {
  using namespace kvip;
  KVIP_REQUIRE(host, "host_unregister: null argument");
  if (cudaHostUnregister(host) != cudaSuccess) return check_launch("cudaHostUnregister");
  return 0;
}

extern "C" uint32_t kvip_streaming_resolver_cores(void) { return 3; }
extern "C" uint32_t kvip_streaming_flag_count(void) { return 16; }
// 2: option bits of this build moved off the reference's flag bits; KvipLiArgs, KvipResolveArgs, KvipFetchArgs and
//    KvipContext grew (wait limit and head-sum mode, source range check and final posts, update status, final posts)
extern "C" uint32_t kvip_b200_abi_version(void) { return 3; }
extern "C" uint32_t kvip_b200_context_bytes(void) { return sizeof(KvipContext); }
extern "C" uint32_t kvip_b200_workspace_bytes(void) { return sizeof(KvipWorkspace); }
extern "C" uint32_t kvip_b200_launch_count(void) { return kvip::g_launches.load(); }
extern "C" const char* kvip_b200_last_error(void) { return kvip::g_error; }

namespace kvip {
namespace {
__global__ void stage_stamp(int64_t* times, uint32_t index, uint32_t copy_previous) {
  uint64_t now;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
  times[index] = copy_previous ? times[index - 1u] : static_cast<int64_t>(now);
}
}  // namespace
}  // namespace kvip

static_assert(sizeof(KvipRuntimeShape) == 80, "runtime shape ABI");
static_assert(sizeof(KvipFinalPost) == 128, "final post ABI (common/lifetch/final_post.h: one cache line)");
static_assert(sizeof(KvipWorkspace) == 256, "workspace ABI");
static_assert(offsetof(KvipWorkspace, options) == 96, "options word lives at byte 96");

extern "C" uint32_t kvip_lifetch_streaming_forward(void* bindings_v, void* update_v, void* workspace_v, void* stream_v,
                                                   const KvipRuntimeShape* shape, uint32_t workers) {
  using namespace kvip;
  KVIP_REQUIRE(bindings_v && update_v && workspace_v && shape, "forward: null blob");
  KVIP_REQUIRE(workers == 1 || workers == 2 || workers == 4, "forward: 1, 2 or 4 fetch workers per query");
  const uint64_t* bind = static_cast<const uint64_t*>(bindings_v);
  const int64_t* upd = static_cast<const int64_t*>(update_v);
  const KvipWorkspace* ws = static_cast<const KvipWorkspace*>(workspace_v);
  const KvipContext* ctx = ptr<const KvipContext>(bind[14]);
  KVIP_REQUIRE(ctx && ptr<const void>(bind[15]) == workspace_v, "forward: bindings do not name this context/workspace");
  KVIP_REQUIRE(std::memcmp(&ctx->shape, shape, sizeof(*shape)) == 0, "forward: shape differs from the bound context");
  KVIP_REQUIRE(ws->history == shape->history && ws->resident == shape->resident && ws->max_events >= KVIP_SLOTS,
               "forward: workspace geometry differs from the shape");
  KVIP_REQUIRE(static_cast<uint64_t>(upd[24]) == shape->history && static_cast<uint64_t>(upd[25]) == shape->resident,
               "forward: update bindings geometry differs from the shape");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const KvipRuntimeShape& s = *shape;
  uint32_t rc;
  KVIP_REQUIRE(!(ws->options & KVIP_OPTION_LEGACY_LAYOUT),
               "forward: the reference's legacy scratch layout (option bit 0x20000000) does not exist in this build");
  // KVIP_OPTION_SCHEDULING_HINTS (parallel finalize, prepare metadata, UBmem overlap) pick between schedules of
  // the reference's pipeline that give the same results: accepted, nothing to do
  const bool select_phase = !(ws->options & KVIP_OPTION_COMMIT_ONLY);
  const bool commit_phase = !(ws->options & KVIP_OPTION_SELECT_ONLY);
  KVIP_REQUIRE(select_phase || commit_phase, "forward: SELECT_ONLY and COMMIT_ONLY exclude each other");
  int64_t* times = (ws->options & KVIP_OPTION_DIAGNOSTICS) ? ptr<int64_t>(ws->times) : nullptr;
  // stamp(i): the stage before boundary i has finished (stream order); skipped = the stage did not run in this call
  auto stamp = [&](uint32_t index, bool skipped) -> uint32_t {
    if (!times) return 0;
    stage_stamp<<<1, 1, 0, stream>>>(times, index, skipped && index ? 1u : 0u);
    count_launch();
    return check_launch("stage_stamp");
  };
  if (select_phase && (rc = stamp(KVIP_TIME_START, false))) return rc;

  KvipLiArgs li{};
  li.query = ptr<const void>(bind[0]); li.keys = ptr<const void>(bind[1]); li.weights = ptr<const void>(bind[2]);
  li.query_scale = ptr<const float>(bind[3]); li.key_scale = ptr<const float>(bind[4]);
  li.key_lengths = ptr<const int32_t>(bind[6]); li.query_ends = ptr<const int32_t>(ctx->query_ends);
  li.block_table = ptr<const int32_t>(bind[7]); li.scores = ptr<float>(bind[12]); li.status = ptr<int32_t>(ws->li_status);
  li.batch = s.batch; li.queries = s.queries; li.heads = s.indexHeads; li.pagesPerRequest = s.pagesPerRequest;
  li.keyRows = s.keyRows; li.scoreStride = s.scoreStride; li.keyDtype = s.keyDtype; li.weightDtype = s.weightDtype;
  li.scoreMode = s.scoreMode; li.ctas = s.smCount;
  KVIP_REQUIRE(li.query && li.keys && li.weights && li.key_lengths && li.query_ends && li.block_table && li.scores && li.status,
               "forward: an LI operand is unbound");
  const bool run_li = select_phase && !(ws->options & KVIP_OPTION_SCORES_READY);
  if (run_li) {
    rc = s.liVariant ? launch_li_score_simt(li, stream) : launch_li_score(li, stream);
    if (rc) return rc;
  }
  if (select_phase && (rc = stamp(KVIP_TIME_LI, !run_li))) return rc;

  KvipTopkArgs tk{};
  tk.scores = li.scores; tk.key_lengths = li.key_lengths; tk.query_ends = li.query_ends;
  tk.topk = ptr<int32_t>(bind[9]); tk.topk_scores = ptr<float>(ws->topk_scores);
  tk.histogram = ptr<uint32_t>(ws->topk_histogram);
  tk.split_scratch = ptr<uint32_t>(ws->topk_split);
  tk.rows = s.batch * s.queries; tk.queries = s.queries; tk.scoreStride = s.scoreStride; tk.base_index = 0;
  KVIP_REQUIRE(tk.topk, "forward: the TopK output is unbound");
  if (select_phase && (rc = launch_topk(tk, stream))) return rc;
  if (select_phase && (rc = stamp(KVIP_TIME_TOPK, false))) return rc;

  KvipResolveArgs rs{};
  rs.topk = tk.topk; rs.row_owners = ptr<const int32_t>(ctx->row_owners); rs.hot_valid = ptr<const int32_t>(ctx->hot_valid);
  rs.reserved_hot = ptr<const int32_t>(ctx->reserved_hot); rs.lru_slots = ptr<const int32_t>(ctx->lru_slots);
  rs.tail_bounds = ptr<const int32_t>(ctx->tail_bounds); rs.logical_ids = ptr<const int64_t>(upd[3]);
  rs.addresses = ptr<const int64_t>(ctx->token_addresses ? ctx->token_addresses : static_cast<uint64_t>(upd[2]));
  rs.locations = ptr<int32_t>(ctx->locations); rs.changes = ptr<int32_t>(ctx->changes);
  rs.change_slots = ptr<int32_t>(ctx->change_slots); rs.change_count = ptr<int32_t>(ctx->change_count);
  rs.events_src = ptr<int32_t>(ws->events_src); rs.events_dst = ptr<int32_t>(ws->events_dst);
  rs.query_counts = ptr<int32_t>(ctx->query_counts); rs.fetch_sources = ptr<int64_t>(ctx->fetch_sources);
  rs.fetch_destinations = ptr<int32_t>(ctx->fetch_destinations);
  rs.logical_output = ptr<int32_t>(upd[22]); rs.slot_output = ptr<int32_t>(upd[23]);
  rs.unpack_indices = ptr<const int64_t>(upd[20]); rs.output_valid = ptr<const int64_t>(upd[21]);
  rs.query_ends = li.query_ends; rs.row_status = ptr<int32_t>(ctx->row_status);
  rs.batch = s.batch; rs.queries = s.queries; rs.history = s.history; rs.resident = s.resident;
  rs.address_stride = static_cast<uint32_t>(ctx->address_stride ? ctx->address_stride : static_cast<uint64_t>(upd[7]));
  rs.outputStride = s.outputStride;
  rs.tokenBytes = s.tokenBytes;
  rs.source_bytes = (ws->options & KVIP_OPTION_DEFERRED_FETCH) ? 0 : ctx->source_bytes;  // descriptors only: the caller fetches
  rs.final_posts = ptr<KvipFinalPost>(ctx->final_posts);
  rs.miss_mask = ptr<uint32_t>(ctx->miss_mask);
  KVIP_REQUIRE(rs.hot_valid && rs.reserved_hot && rs.lru_slots && rs.logical_ids && rs.addresses && rs.locations &&
                   rs.changes && rs.change_slots && rs.change_count && rs.events_src && rs.events_dst && rs.query_counts &&
                   rs.fetch_sources && rs.fetch_destinations && rs.row_status, "forward: a resolver operand is unbound");
  KVIP_REQUIRE(rs.tail_bounds == nullptr || (s.outputStride - s.resident >= 384 && (s.outputStride - s.resident) % 128 == 0),
               "forward: ABC tail bounds need at least 384 dedicated output slots behind the hot ones, in blocks of 128");
  if (select_phase && (rc = launch_resolve_requests(rs, stream))) return rc;
  if (select_phase && (rc = stamp(KVIP_TIME_RESOLVE, false))) return rc;
  if (!commit_phase) return 0;

  // ---- commit phase: service outputs, Index exchange, fetch, gather ----------------------------------------
  // Serial (default): all on `stream`, in that order. Overlapped (side stream, two events and the miss mask bound):
  //     stream      : fork ................ fetch (copies only) ...... join -> publish residency -> gather(misses)
  //     side stream :      outputs -> exchange -> gather(hits) -> join
  // The fetch of a step with misses is bound by the host link and leaves HBM idle; the exchange and the gather of
  // the entries that were hits touch neither the victim slots nor the fetch descriptors, so they run beside it.
  // Residency is published after BOTH the exchange (which revokes freed positions) and the fetch have finished.
  const bool fetch_runs = !(ws->options & KVIP_OPTION_DEFERRED_FETCH);
  const bool overlapped = fetch_runs && ws->side_stream && ws->fork_event && ws->join_event && ctx->miss_mask && !ws->staging;
  cudaStream_t side = overlapped ? reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(ws->side_stream)) : stream;
  cudaEvent_t fork_event = reinterpret_cast<cudaEvent_t>(static_cast<uintptr_t>(ws->fork_event));
  cudaEvent_t join_event = reinterpret_cast<cudaEvent_t>(static_cast<uintptr_t>(ws->join_event));
  auto stamp_on = [&](cudaStream_t where, uint32_t index, bool skipped) -> uint32_t {
    if (!times) return 0;
    stage_stamp<<<1, 1, 0, where>>>(times, index, skipped && index ? 1u : 0u);
    count_launch();
    return check_launch("stage_stamp");
  };
  if (overlapped) {
    if (cudaEventRecord(fork_event, stream) != cudaSuccess || cudaStreamWaitEvent(side, fork_event, 0) != cudaSuccess)
      return check_launch("forward: forking the side stream");
  }
  if ((rc = launch_publish_outputs(rs, side))) return rc;
  if ((rc = stamp_on(side, KVIP_TIME_OUTPUTS, false))) return rc;
  if (ws->slots_ready_event &&
      cudaEventRecord(reinterpret_cast<cudaEvent_t>(static_cast<uintptr_t>(ws->slots_ready_event)), side) != cudaSuccess)
    return check_launch("forward: recording the slots-ready event");

  KvipExchangeArgs ex{};
  ex.keys = ptr<uint8_t>(upd[0]); ex.scales = ptr<float>(upd[1]); ex.addresses = ptr<int64_t>(upd[2]);
  ex.logical_ids = ptr<int64_t>(upd[3]); ex.hot_valid = ptr<int32_t>(upd[16]);
  ex.events_src = rs.events_src; ex.events_dst = rs.events_dst; ex.query_counts = rs.query_counts;
  ex.row_owners = rs.row_owners; ex.row_status = rs.row_status; ex.shadow = ptr<uint32_t>(ws->dense_shadow);
  ex.status = ptr<int32_t>(upd[6]);
  ex.batch = s.batch; ex.queries = s.queries; ex.history = s.history; ex.resident = s.resident;
  ex.address_stride = static_cast<uint32_t>(upd[7]); ex.key_row_bytes = s.keyDtype == KVIP_KEY_BF16 ? 256u : 128u;
  KVIP_REQUIRE(ex.keys && ex.scales && ex.addresses && ex.hot_valid && ex.shadow && ex.status, "forward: an update operand is unbound");
  if ((rc = launch_exchange(ex, side))) return rc;
  if ((rc = stamp_on(side, KVIP_TIME_EXCHANGE, false))) return rc;

  if (!fetch_runs) {  // deferred fetch: descriptors only
    if ((rc = stamp(KVIP_TIME_FETCH, true))) return rc;
    return stamp(KVIP_TIME_GATHER, true);
  }
  KvipFetchArgs ft{};
  ft.source_base = ptr<const uint8_t>(ctx->source_base); ft.fetch_sources = rs.fetch_sources;
  ft.fetch_destinations = rs.fetch_destinations; ft.query_counts = rs.query_counts; ft.row_owners = rs.row_owners;
  ft.row_status = rs.row_status; ft.pool = ptr<uint8_t>(ctx->pool); ft.hot_valid = ex.hot_valid;
  ft.source_bytes = ctx->source_bytes; ft.batch = s.batch; ft.resident = s.resident; ft.outputStride = s.outputStride;
  ft.tokenBytes = s.tokenBytes; ft.status = ex.status; ft.defer_publication = overlapped ? 1u : 0u;
  KVIP_REQUIRE(ft.source_base && ft.pool, "forward: the KV pools are unbound");
  KvipGatherArgs ga{};
  const bool gathers = s.gatherRows && ws->gather_out;
  ga.pool = ft.pool; ga.slots = rs.locations; ga.row_owners = rs.row_owners; ga.out = ptr<uint8_t>(ws->gather_out);
  ga.rows = s.batch * s.queries; ga.queries = s.queries; ga.outputStride = s.outputStride; ga.tokenBytes = s.tokenBytes;
  if (!overlapped) {
    if ((rc = ws->staging ? launch_fetch_staged(ft, *ws, stream) : launch_fetch(ft, stream))) return rc;
    if ((rc = stamp(KVIP_TIME_FETCH, false))) return rc;
    if (gathers && (rc = launch_gather(ga, stream))) return rc;
    return stamp(KVIP_TIME_GATHER, !gathers);
  }
  ga.miss_mask = rs.miss_mask;
  if (gathers) {
    ga.phase = 1u;   // entries that were hits: beside the fetch
    if ((rc = launch_gather(ga, side))) return rc;
  }
  if (cudaEventRecord(join_event, side) != cudaSuccess) return check_launch("forward: recording the join event");
  if ((rc = launch_fetch(ft, stream))) return rc;
  if ((rc = stamp(KVIP_TIME_FETCH, false))) return rc;
  if (cudaStreamWaitEvent(stream, join_event, 0) != cudaSuccess) return check_launch("forward: joining the side stream");
  if ((rc = launch_publish_residency(ft, stream))) return rc;
  if (gathers) {
    ga.phase = 2u;   // entries the fetch has just filled
    if ((rc = launch_gather(ga, stream))) return rc;
  }
  return stamp(KVIP_TIME_GATHER, !gathers);
}
