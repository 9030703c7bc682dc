/* C ABI of libkvip_b200.so: the DeepSeek-sparse-attention selection-and-fetch path
 * (lightning-indexer score -> TopK-2048 -> slot resolver -> KV fetch -> Index update)
 * as hand-written CUDA for sm_100a.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; no torch types;
 *   - every pointer inside an argument struct is a DEVICE pointer unless the field
 *     comment says "host";
 *   - `stream` is a cudaStream_t passed as void*; work is only enqueued, nothing
 *     synchronises, allocates or copies to the host;
 *   - return value 0 = enqueued, 100000 = bad argument (the reference's launch
 *     convention, csrc/operators/lightning_indexer_with_fetch/op_host/launch.cpp:77-78),
 *     any other value = 200000 + cudaError_t of the failed launch;
 *   - device-side failures are reported through int32 status words, never by a trap.
 *
 * Citations name files of the reference project (zxdgongjue-spec/KVIP) by their
 * path inside that project.
 */
#ifndef KVIP_B200_H_
#define KVIP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVIP_TOPK 2048u              /* context.h:6 kTop */
#define KVIP_MAX_QUERIES 4u          /* adapters/vllm/inputs.py:11 */
#define KVIP_SLOTS 8192u             /* context.h:6 kSlots = 4 * 2048 */
#define KVIP_LRU_SLOTS 2048u         /* common/lifetch/cache_metadata.h:2 */
#define KVIP_CHANGE_CAPACITY 10240u  /* common/lifetch/cache_metadata.h:3 */
#define KVIP_BLOCK_TOKENS 128u       /* paged Index cache block */
#define KVIP_INDEX_WIDTH 128u        /* d_I */
#define KVIP_TOPK_SPLIT_WORDS 20544u /* u32 words of TopK scratch per score row for the multi-CTA path */
/* Bits of KvipWorkspace.options. Bits 0-15: prefetch limit, 16-18: fetch workers per query, both as the
 * reference packs them (python/kvip/operators/lifetch/streaming.py:133-146). The reference's own flag bits keep
 * their positions: diagnostics and deferred fetch mean what they mean there; parallel finalize (0x10000000),
 * prepare metadata (0x08000000) and UBmem overlap (0x04000000) choose between schedules of the Ascend pipeline
 * that give the same results, so they are accepted and have no effect here; the legacy scratch layout
 * (0x20000000) cannot be honoured and is rejected with KVIP_BAD_ARGUMENT. The bits this build adds sit where
 * the reference has none. */
#define KVIP_OPTION_DIAGNOSTICS 0x80000000u    /* device timestamps of every stage into KvipWorkspace.times */
#define KVIP_OPTION_DEFERRED_FETCH 0x40000000u /* descriptors only: no fetch, no gather */
#define KVIP_OPTION_LEGACY_LAYOUT 0x20000000u  /* reference only: rejected */
#define KVIP_OPTION_SCHEDULING_HINTS 0x1c000000u /* reference only: accepted, no effect */
#define KVIP_OPTION_SELECT_ONLY 0x02000000u    /* LI score -> TopK -> resolver, then return */
#define KVIP_OPTION_COMMIT_ONLY 0x01000000u    /* the rest of a SELECT_ONLY call: outputs -> exchange -> fetch (-> gather) */
#define KVIP_OPTION_SCORES_READY 0x00800000u   /* the score rows were written by earlier launches: the select phase starts at TopK */
#define KVIP_BAD_ARGUMENT 100000u
#define KVIP_CUDA_ERROR_BASE 200000u

/* device status bits (row_status / update.status words) */
#define KVIP_ERR_TOKEN_RANGE 1u      /* selected position >= history (resolver_staged_dma2.h:63) */
#define KVIP_ERR_NO_SLOT 4u          /* victims exhausted / bad candidate (resolver_staged_dma2.h:150,185) */
#define KVIP_ERR_HASH 8u             /* hash probe overflow, also the wait-limit code (streaming.cpp:191) */
#define KVIP_ERR_EXCHANGE 16u        /* Index exchange plan invalid (shadow_exchange_parallel.h:40) */
#define KVIP_ERR_PIPELINE 32u        /* a bounded mbarrier wait inside the LI kernel gave up */
#define KVIP_ERR_SOURCE 64u          /* a missing row's source address lies outside the host pool (streaming.cpp:399-400) */
#define KVIP_ERR_PEER 128u           /* a bounded wait for another GPU's candidates gave up (sequence-sharded TopK) */

enum { KVIP_KEY_FP8_E4M3 = 0, KVIP_KEY_BF16 = 1 };
enum { KVIP_WEIGHT_BF16 = 0, KVIP_WEIGHT_FP32 = 1 };
enum { KVIP_SCORE_FP32 = 0, KVIP_SCORE_BF16_AWAY = 1 };

/* Geometry bound before graph capture. Same size (80 bytes, 20 x u32) and the same
 * leading fields as rotating::RuntimeShape (include/runtime_shape.h:5-27); the fields
 * that described Ascend core scheduling carry the CUDA tiling instead. */
typedef struct KvipRuntimeShape {
  uint32_t batch;          /* requests per launch (reference limit 16 lifted) */
  uint32_t history;        /* Index positions per owner, multiple of 128 */
  uint32_t resident;       /* hot KV slots per owner, multiple of 128, >= 2048 */
  uint32_t indexHeads;     /* 32 or 64 */
  uint32_t smCount;        /* persistent CTAs for the LI kernel (0 = query the device) */
  uint32_t queries;        /* query slots per request, 1..4 */
  uint32_t keyDtype;       /* KVIP_KEY_* */
  uint32_t weightDtype;    /* KVIP_WEIGHT_* */
  uint32_t scoreMode;      /* KVIP_SCORE_* */
  uint32_t pagesPerRequest;/* derived: history / 128 */
  uint32_t finalWorkers;   /* kept for ABI parity, always 4 */
  uint32_t scoreStride;    /* derived: floats per score row (= history) */
  uint32_t outputStride;   /* KV slots per owner in the resident pool (0 -> resident) */
  uint32_t owners;         /* stable owners in the Index storage (0 -> batch) */
  uint32_t tokenBytes;     /* bytes per KV row, multiple of 16 (same index as the reference) */
  uint32_t keyRows;        /* rows of the paged key tensor = owners * history */
  uint32_t gatherRows;     /* 1 = also write the dense [T,2048,tokenBytes] gather */
  uint32_t liVariant;      /* 0 = tcgen05 kernel, 1 = CUDA-core cross-check kernel */
  uint32_t reserved0;
  uint32_t reserved1;
} KvipRuntimeShape;

/* ---- stage 1: lightning-indexer score ------------------------------------------
 * score[t,s] = kscale[s] * sum_h W[t,h] * relu(q[t,h,:] . k[s,:]),
 * W = float(w) * qscale (bf16 weights) or W = w (fp32 weights).
 * Replaces QLIMatmul::ComputeMm1 + the score epilogue
 * (op_kernel/indexer/indexer_cube.h:161-322, indexer_score.h:59-140,384-426). */
typedef struct KvipLiArgs {
  const void* query;          /* [batch*queries, heads, 128] fp8 e4m3 or bf16 */
  const void* keys;           /* [keyRows, 128] paged, 128-token blocks */
  const void* weights;        /* [batch*queries, heads] bf16 or fp32 */
  const float* query_scale;   /* [batch*queries, heads] or NULL (= 1) */
  const float* key_scale;     /* [keyRows] or NULL (= 1) */
  const int32_t* key_lengths; /* [batch] */
  const int32_t* query_ends;  /* [batch, queries] exclusive causal bound, 0 = padding row */
  const int32_t* block_table; /* [batch, pagesPerRequest] page -> 128-row block of keys */
  float* scores;              /* [batch*queries, scoreStride] */
  int32_t* status;            /* [1] OR-ed KVIP_ERR_* */
  uint32_t batch, queries, heads, pagesPerRequest;
  uint32_t keyRows, scoreStride, keyDtype, weightDtype;
  uint32_t scoreMode, ctas;
  uint32_t stages;            /* key pages in flight per CTA; 0 = as many as shared memory holds */
  uint32_t withhold_tile;     /* test hook for the bounded waits: when n > 0, CTA 0 never loads its n-th key page,
                                 so the wait for that page runs out and the kernel returns with
                                 KVIP_ERR_PIPELINE in *status; 0 in production */
  uint32_t wait_kilocycles;   /* limit of every barrier wait inside the kernel, in units of 1024 SM clock cycles;
                                 0 = the default of about one second */
  uint32_t reserved0;
} KvipLiArgs;
uint32_t kvip_b200_li_score(const KvipLiArgs* args, void* stream);
/* CUDA-core restatement of the same formula with the oracle's accumulation order;
 * an on-GPU cross-check for small shapes, not the product path. */
uint32_t kvip_b200_li_score_simt(const KvipLiArgs* args, void* stream);

/* ---- stage 2: per-query TopK-2048 -----------------------------------------------
 * Valid length L = min(key_length[b], query_end[t]); L<=0 -> 2048 x -1; L<2048 ->
 * 0..L-1 then -1; otherwise every position with key > v (v = 2048th largest) in
 * ascending position, then positions with key == v in ascending position, cut at 2048.
 * Replaces LITopk / LiTopKVF (op_kernel/indexer/topk.h:155-187,
 * topk_common.h:1136-1187; bounds indexer_vector.h:826-957). */
typedef struct KvipTopkArgs {
  const float* scores;        /* [rows, scoreStride] */
  const int32_t* key_lengths; /* [batch] */
  const int32_t* query_ends;  /* [batch*queries] */
  int32_t* topk;              /* [rows, 2048] */
  float* topk_scores;         /* [rows, 2048] or NULL: score of each output */
  uint32_t* histogram;        /* [rows, 4096] all-zero scratch (left all-zero) or NULL: with it the first
                                 radix pass runs on the whole GPU in a kernel of its own */
  uint32_t rows, queries, scoreStride, base_index; /* base_index added to every output index */
  uint32_t* split_scratch;    /* [rows, KVIP_TOPK_SPLIT_WORDS] scratch or NULL: with it every pass runs on several
                                 CTAs per row (takes precedence over `histogram`). The first 4160 words of each
                                 row must be zero on entry and are zero again on return. */
} KvipTopkArgs;
uint32_t kvip_b200_topk(const KvipTopkArgs* args, void* stream);

/* Same selection for callers that cannot allocate device memory (for instance a serving process whose
 * KV-cache pool already owns all free HBM, or a decode-loop plugin that must not stall the device on an
 * allocation). No counterpart in the reference. `histogram` of the argument struct is ignored: the
 * [rows, 4096] scratch is a 4 MiB array inside the library image, held by every GPU that loads the
 * library until the process exits. Limit: rows <= 256 (KVIP_BAD_ARGUMENT with a message beyond that).
 * The call allocates nothing; it clears the rows of the scratch it is about to use on `stream` first.
 * The first call on a device looks up the scratch address (a one-time set-up): make that first call
 * before any stream capture. All calls share the one array: calls that overlap on the GPU (different
 * streams, or different threads) race on it - keep them on one stream. */
uint32_t kvip_b200_topk_static(const KvipTopkArgs* args, void* stream);

/* Merge of sequence-sharded candidates: rows x shards x 2048 (score,index) pairs ->
 * global top-2048 under the same total order. New on B200 (no reference counterpart;
 * precedent: the on-chip sequence split, common/lifetch/sequence_schedule.h:9-37). */
typedef struct KvipMergeArgs {
  const float* cand_scores;   /* [rows, shards*2048], or any layout the two strides describe */
  const int32_t* cand_index;  /* same layout, -1 = empty */
  int32_t* topk;              /* [rows, 2048] */
  uint32_t rows, shards;
  uint32_t shard_stride;      /* elements between the candidate lists of two shards of one row; 0 = 2048 */
  uint32_t row_stride;        /* elements between two rows of one shard; 0 = shards * 2048. The buffer an all-gather of
                                 per-rank [2, rows, 2048] (scores, indices) blocks fills is read in place with
                                 shard_stride = 2 * rows * 2048 and row_stride = 2048. */
  /* Candidates delivered by kvip_b200_peer_exchange instead of the three pointers above (all optional, NULL / 0 =
   * unused): `peer_block` is this rank's exchange block. The kernel reads the block's step counter, waits (bounded) until
   * the flags of `wait_ranks` ranks have reached it, and merges the candidates of that step's half of the block. A wait
   * that runs out ORs KVIP_ERR_PEER into *status and the rows come back as -1. */
  const void* peer_block;
  int32_t* status;
  uint32_t wait_ranks;        /* = shards when peer_block is set */
  uint32_t wait_kilocycles;   /* limit of the wait in units of 1024 SM clock cycles; 0 = about one second */
} KvipMergeArgs;
uint32_t kvip_b200_topk_merge(const KvipMergeArgs* args, void* stream);

/* ---- exchange of the per-rank TopK candidates over NVLink peer memory --------------------------
 * The one exchange step of a sequence-sharded request (every rank's 2048 (score, index) candidates per row to every
 * rank) written as a kernel of this library instead of an NCCL all-gather: 16 KiB per rank is pure latency, a
 * collective library's launch and synchronisation cost several times the transfer, and a plain kernel can live in the
 * same CUDA graph as the score and TopK kernels on either side. One process per GPU; no two ranks may share a GPU
 * (the merge kernel of one rank waits for the exchange kernel of the others).
 *
 * Every rank owns one exchange block (kvip_b200_peer_alloc; cudaMalloc'ed, zeroed, with an IPC handle that the other
 * ranks open with kvip_b200_peer_open):
 *   bytes    0..255   step counter (u32) of this rank: the number of exchanges it has made
 *   bytes  256..511   flags[8] (u32): flags[r] = last step whose candidates rank r has delivered HERE
 *   bytes  512..      two halves (step parity) x world x block_bytes: the candidate blocks, in rank order
 * kvip_b200_peer_exchange (one CTA): step s = counter + 1; copies `send` (block_bytes, a multiple of 16) into slot
 * [s & 1][rank] of every rank's block with plain peer stores, fences system-wide, then writes s into flags[rank] of
 * every rank and into its own counter. Two halves suffice: a rank starts exchange s + 2 only after its merge of step
 * s + 1, which has seen every rank's flag s + 1, which every rank wrote after its own merge of step s. */
#define KVIP_PEER_HEADER_BYTES 512u
typedef struct KvipPeerExchangeArgs {
  const void* send;           /* this rank's candidates: [2, rows, 2048] int32 (score bits, indices) */
  uint64_t peer_block[8];     /* exchange block of every rank as mapped in THIS process (own block at [rank]) */
  uint32_t block_bytes;       /* bytes of `send` */
  uint32_t rank, world, reserved0;
} KvipPeerExchangeArgs;
uint32_t kvip_b200_peer_exchange(const KvipPeerExchangeArgs* args, void* stream);
/* Exchange block of `bytes` (>= 512 + 2 * world * block_bytes) on the current device, zeroed; `handle` receives the
 * 64-byte CUDA IPC handle that other processes pass to kvip_b200_peer_open. */
uint32_t kvip_b200_peer_alloc(uint64_t bytes, void** block, uint8_t* handle);
uint32_t kvip_b200_peer_open(const uint8_t* handle, void** block);   /* maps another rank's block (enables peer access) */
uint32_t kvip_b200_peer_close(void* block);                           /* a mapping made by kvip_b200_peer_open */
uint32_t kvip_b200_peer_free(void* block);                            /* a block made by kvip_b200_peer_alloc */

/* ---- QueryInputs.pack / bind_positions ---------------------------------------------------
 * Row r of the bound input buffers takes token gather_indices[r] of the caller's tensors; query_ends[r] =
 * (positions[token] + 1) * query_valid[r]. Any of the three source groups may be NULL (skipped). One launch
 * instead of the index_select / add / mul / copy calls of the reference (adapters/vllm/inputs.py:121-152). */
typedef struct KvipPackArgs {
  const uint8_t* query_src;     /* [tokens, query_row_bytes] or NULL */
  const uint8_t* weights_src;   /* [tokens, weights_row_bytes] or NULL */
  const float* scale_src;       /* [tokens, heads] or NULL */
  const int64_t* positions_src; /* [tokens] or NULL */
  const int64_t* gather_indices;/* [rows] */
  const int64_t* query_valid;   /* [rows] 0/1 */
  uint8_t* query_dst;           /* [rows, query_row_bytes] */
  uint8_t* weights_dst;         /* [rows, weights_row_bytes] */
  float* scale_dst;             /* [rows, heads] */
  int64_t* position_scratch;    /* [rows] */
  int32_t* query_ends;          /* [rows] */
  uint32_t rows, tokens, heads, query_row_bytes, weights_row_bytes, reserved0;
} KvipPackArgs;
uint32_t kvip_b200_pack_inputs(const KvipPackArgs* args, void* stream);

/* ---- resident threshold and cold predicate ---------------------------------------------
 * Input: the TopK of the RESIDENT prefix of every score row (kvip_b200_topk run with the row's query end
 * clipped to `resident`) with its scores. Output per row: the threshold key (order-preserving u32 image of the
 * smallest selected score; 0 while the prefix holds fewer than 2048 valid positions), one bit per cold
 * position (position resident + 32 w + i is bit i of word w) set when its score beats the threshold, and the
 * number of set bits. The marked positions contain the cold part of the row's final TopK: they are the
 * candidates of a speculative prefetch. Replaces ProcessResidentTopK / SaveResident / ClassifyScore /
 * BatchClassifyScore (op_kernel/indexer/indexer_vector.h:100-105, 162-234; indexer_score.h:784-792, 976-1017);
 * the forward of this build does not consume it. */
typedef struct KvipColdArgs {
  const float* scores;          /* [rows, scoreStride] */
  const int32_t* key_lengths;   /* [rows / queries] */
  const int32_t* query_ends;    /* [rows] */
  const int32_t* prefix_topk;   /* [rows, 2048] TopK of positions < resident, -1 padded */
  const float* prefix_scores;   /* [rows, 2048] their scores */
  uint32_t* threshold_keys;     /* [rows] out */
  uint32_t* bitmap;             /* [rows, bitmap_words] out */
  int32_t* counts;              /* [rows] out */
  uint32_t rows, queries, scoreStride, resident, bitmap_words, reserved0;
} KvipColdArgs;
uint32_t kvip_b200_cold_predicate(const KvipColdArgs* args, void* stream);

/* ---- stage 3: classification + resolver + service outputs + fetch descriptors ---
 * Replaces ClassifyTopkHalf / StagedInitializeReady / StagedQuery / PackStagedUrmaQuery /
 * PublishQueryOutputs (op_kernel/staged_topk_classify.h:9-46,
 * resolver_staged_dma2.h:83-237, staged_urma_pack.h:6-71, streaming.cpp:66-90).
 *
 * ABC tail (common/lifetch/cache_metadata.h:22-26, 100-105; prefetch.h:26-44): with tail_bounds bound, the
 * positions [begin, end) of a request are tokens written since the last commit to the host pool. Their KV rows
 * live in a ring of outputStride - resident dedicated slots behind the hot slots. Such a position is never a hot
 * hit by position, never a miss and never a victim: while begin <= p < begin + ring size its location is
 * resident + p % ring size (the reference stores the code resident + 8192 + p % ring in its mapping and resolves
 * it to the same slot); a tail position beyond the ring is resolved like any cold position.
 *
 * Final posts (common/lifetch/final_post.h:2-12; include/context.h:9-14): one 128-byte record per (request, query)
 * = 32 x u32 {count, pending, error, deferred, descriptor, nonconflicting, head lo, head hi, 0...}: count = new
 * slots of the query, descriptor = index of its first descriptor in fetch_sources / fetch_destinations
 * (request * 8192 + descriptors of the earlier queries; the reference gives every query a fixed 2048-entry
 * region instead), nonconflicting = count (no prefetch ever writes a victim slot in this build, so every
 * descriptor is safe to fetch at once), error = the request's status word, pending = deferred = head = 0. */
typedef struct KvipFinalPost {
  uint32_t count, pending, error, deferred, descriptor, nonconflicting;
  uint32_t head_lo, head_hi;
  uint32_t reserved[24];
} KvipFinalPost;
typedef struct KvipResolveArgs {
  const int32_t* topk;          /* [batch, queries, 2048] selected physical positions */
  const int32_t* row_owners;    /* [batch] or NULL (owner = row) */
  const int32_t* hot_valid;     /* [owners, resident] */
  const int32_t* reserved_hot;  /* [batch, resident] candidate ordinal or -1 */
  const int32_t* lru_slots;     /* [batch, 2048] victim candidates, oldest first */
  const int32_t* tail_bounds;   /* [batch, 2] or NULL */
  const int64_t* logical_ids;   /* [owners, history] (pre-update ids) */
  const int64_t* addresses;     /* [owners, address_stride] source address of each position */
  int32_t* locations;           /* [batch, queries, 2048] out */
  int32_t* changes;             /* [batch, 10240] out: token per record, -1 = none */
  int32_t* change_slots;        /* [batch, 10240] out */
  int32_t* change_count;        /* [batch] out: 2048 + new slots */
  int32_t* events_src;          /* [batch, 8192] out: position per new slot, rank order */
  int32_t* events_dst;          /* [batch, 8192] out */
  int32_t* query_counts;        /* [batch, 8]: [0..3] new slots per query, [4] total */
  int64_t* fetch_sources;       /* [batch, 8192] out: address snapshot per new slot */
  int32_t* fetch_destinations;  /* [batch, 8192] out: owner*outputStride + slot */
  int32_t* logical_output;      /* [batch*queries, 2048] or NULL */
  int32_t* slot_output;         /* [batch*queries, 2048] or NULL */
  const int64_t* unpack_indices;/* [batch*queries] output row -> source query row, or NULL (identity) */
  const int64_t* output_valid;  /* [batch*queries] 0 = padding output row (-1 fill), or NULL */
  const int32_t* query_ends;    /* [batch*queries]; rows with 0 publish -1 when no routing is bound */
  int32_t* row_status;          /* [batch, 32] */
  uint32_t batch, queries, history, resident;
  uint32_t address_stride, outputStride;
  uint32_t tokenBytes;          /* bytes per KV row: with source_bytes, the range check of the source addresses */
  uint32_t reserved1;
  uint64_t source_bytes;        /* size of the miss source; 0 = addresses are not checked here */
  KvipFinalPost* final_posts;   /* [batch, 4] out, or NULL */
  uint32_t* miss_mask;          /* [batch*queries, 64] out or NULL: bit k of a row = entry k of that TopK row was a miss
                                   (its slot is filled by this round's fetch); lets the gather run in two phases */
} KvipResolveArgs;
uint32_t kvip_b200_resolve(const KvipResolveArgs* args, void* stream);

/* ---- stage 4: fetch ----------------------------------------------------------------
 * output[dest*tokenBytes : +tokenBytes] = source_base[address : +tokenBytes] for every
 * descriptor, then hot_valid[owner, slot] = 1. The source is the device alias of a
 * pinned, mapped host pool (or any device-visible memory). Replaces FetchQueryGroup ->
 * kvaf_device::KvafBatchGetDevice (streaming.cpp:365-500; arithmetic in
 * patches/kvaf-ubmem-device-get.patch, fused_batch_get_device.h:21-61) and
 * PublishQueryCompletion (streaming.cpp:300-328). */
typedef struct KvipFetchArgs {
  const uint8_t* source_base;      /* device-visible base the addresses are relative to */
  const int64_t* fetch_sources;    /* [batch, 8192] byte offsets from source_base */
  const int32_t* fetch_destinations;/* [batch, 8192] row index into pool */
  const int32_t* query_counts;     /* [batch, 8], word 4 = descriptors of the request */
  const int32_t* row_owners;       /* [batch] or NULL */
  int32_t* row_status;             /* [batch, 32]; a failed request moves nothing; word 2 = fetch error */
  uint8_t* pool;                   /* [owners*outputStride, tokenBytes] resident KV pool */
  int32_t* hot_valid;              /* [owners, resident] */
  uint64_t source_bytes;           /* size of the source window, for the bounds check */
  uint32_t batch, resident, outputStride, tokenBytes;
  int32_t* status;                 /* [batch] Index-update status or NULL: a descriptor that fails the range check
                                      ORs 4 into its request's word (index_cache_update.h:6-20) and the destination
                                      slot loses residency, so the next step cannot read a stale row as a hit */
  uint32_t defer_publication;      /* 1 = copy only; hot_valid = 1 is left to kvip_b200_publish_residency */
  uint32_t reserved0;
} KvipFetchArgs;
uint32_t kvip_b200_fetch(const KvipFetchArgs* args, void* stream);
/* hot_valid[owner, slot] = 1 for every descriptor the fetch accepted (same argument struct, same checks). Split from
 * the copy for callers that run the fetch beside the Index exchange: the exchange revokes the residency of
 * positions it frees, and a slot freed there and refilled by this round's fetch must end up valid, so the
 * publication has to come after both (PublishQueryCompletion, streaming.cpp:300-328, has the same order). */
uint32_t kvip_b200_publish_residency(const KvipFetchArgs* args, void* stream);

/* Dense gather of the selected rows: out[t, k, :] = pool[owner*outputStride + slot[t,k], :],
 * zero rows where slot < 0. (The north-star "fetch" output; the reference hands slot
 * indices to its attention kernel instead, streaming.cpp:66-90.) */
typedef struct KvipGatherArgs {
  const uint8_t* pool;
  const int32_t* slots;        /* [rows, 2048] */
  const int32_t* row_owners;   /* [batch] or NULL */
  uint8_t* out;                /* [rows, 2048, tokenBytes] */
  uint32_t rows, queries, outputStride, tokenBytes;
  const uint32_t* miss_mask;   /* [rows, 64] from the resolver, or NULL */
  uint32_t phase;              /* with miss_mask: 0 = every entry, 1 = only entries that were hits (independent of this
                                  round's fetch), 2 = only entries that were misses */
  uint32_t reserved0;
} KvipGatherArgs;
uint32_t kvip_b200_gather(const KvipGatherArgs* args, void* stream);

/* ---- stage 5: Index exchange (hot-slot permutation) -------------------------------
 * Applies the (position, slot) events of one round so that physical position p < resident
 * describes hot slot p. Replaces ApplyBatch/ApplyDenseBatch/Commit*Metadata
 * (op_kernel/shadow_exchange_parallel.h:27-198; driver streaming.cpp:205-274). */
typedef struct KvipExchangeArgs {
  uint8_t* keys;               /* [owners, history, 128] (row bytes = 128 * key element size) */
  float* scales;               /* [owners, history] */
  int64_t* addresses;          /* [owners, address_stride] */
  int64_t* logical_ids;        /* [owners, history] */
  int32_t* hot_valid;          /* [owners, resident] */
  const int32_t* events_src;   /* [batch, 8192] */
  const int32_t* events_dst;   /* [batch, 8192] */
  const int32_t* query_counts; /* [batch, 8] */
  const int32_t* row_owners;   /* [batch] or NULL */
  const int32_t* row_status;   /* [batch, 32] or NULL: word 0 != 0 -> the request failed upstream */
  uint32_t* shadow;            /* [batch, 2*history] identity maps, restored on exit */
  int32_t* status;             /* [batch] update status */
  uint32_t batch, queries, history, resident;
  uint32_t address_stride, key_row_bytes, reserved0, reserved1;
} KvipExchangeArgs;
uint32_t kvip_b200_exchange(const KvipExchangeArgs* args, void* stream);

/* ---- paged Index-cache update (new tokens) -----------------------------------------
 * keys[owner, query_end-1] = src[slot_mapping[gather[row]]], same for scales; invalid rows
 * write row `row` of owner 0. With bf16 sources the row is quantised to FP8 e4m3 with a
 * per-token scale amax/448. Replaces VllmIndexCacheStorage.ingest_decode
 * (python/kvip/adapters/vllm/index_import.py:38-52). */
typedef struct KvipIngestArgs {
  const void* source_keys;       /* [source_rows, 128] u8 (fp8) or bf16 */
  const float* source_scales;    /* [source_rows] or NULL when quantising */
  const int64_t* slot_mapping;   /* [tokens] */
  const int64_t* gather_indices; /* [batch*queries] */
  const int32_t* query_ends;     /* [batch*queries] */
  const int32_t* row_owners;     /* [batch] */
  uint8_t* keys;                 /* [owners, history, 128] */
  float* scales;                 /* [owners, history] */
  uint32_t batch, queries, history, source_is_bf16;
} KvipIngestArgs;
uint32_t kvip_b200_ingest(const KvipIngestArgs* args, void* stream);

/* Prefill-side import of Index rows: one launch for every request of a forward batch
 * (VllmIndexCacheStorage.ingest_prefill, python/kvip/adapters/vllm/index_import.py:17-36, does it with
 * index_select / index_copy_ calls per request). A span of kind 0 restores a request's cached history: Index
 * position p in [first, first + tokens) of `owner` takes cache row block_table[row, p / block] * block + p % block.
 * A span of kind 1 writes the tokens of this forward: batch token t in [first, first + tokens) goes to Index
 * position positions[t] of `owner` from cache row slot_mapping[t]. Rows whose source or target is out of range
 * are skipped and counted in *errors. */
typedef struct KvipIngestSpanArgs {
  const uint8_t* source_keys;    /* [source_rows, 128] FP8 rows of the model's paged cache */
  const float* source_scales;    /* [source_rows] */
  const int32_t* block_table;    /* [table_rows, table_stride] */
  const int64_t* slot_mapping;   /* [batch_tokens] */
  const int64_t* positions;      /* [batch_tokens] */
  const int32_t* spans;          /* [count, 8]: owner, table row, kind, first, tokens, 0, 0, 0 */
  uint8_t* keys;                 /* [owners, history, 128] */
  float* scales;                 /* [owners, history] */
  int32_t* errors;               /* [1] in/out or NULL */
  uint64_t source_rows;
  uint32_t count, max_tokens, owners, history;
  uint32_t block, table_rows, table_stride, batch_tokens;
} KvipIngestSpanArgs;
uint32_t kvip_b200_ingest_spans(const KvipIngestSpanArgs* args, void* stream);

/* ---- SlotLRU commit on the device -------------------------------------------------
 * Same list semantics as _commit_lru_rows / _write_oldest_victims
 * (python/kvip/cache/_lru_kernel.py:32-199): unique touched slots move to the tail in
 * ascending slot order, then the first min(2048, active) nodes are listed as victims.
 * The list is held as an array (`order`, oldest first) instead of next/previous links, so
 * a commit is one parallel stream compaction per row; `reserved_hot` is rewritten as the
 * inverse of the victim list. One CTA per row. */
typedef struct KvipLruArgs {
  int32_t* order;              /* [rows, capacity] slots, oldest first; in/out */
  int32_t* slots;              /* [rows, 2048] victims; in (previous victims) / out */
  int32_t* bitmap;             /* [rows, words] out: victim bitmap (also dedup scratch) */
  int32_t* unique;             /* [rows] out: distinct touched slots */
  int32_t* reserved_hot;       /* [rows, resident] in/out or NULL */
  const int32_t* touched;      /* [rows, touched_stride] slots; <0 or >= active ignored */
  const int32_t* active;       /* [rows] committed slots in the list */
  uint32_t rows, capacity, words, touched_stride;
  uint32_t resident, reserved0, reserved1, reserved2;
} KvipLruArgs;
uint32_t kvip_b200_lru_commit(const KvipLruArgs* args, void* stream);

/* ---- ABC tail maps (python/kvip/cache/abc.py:5-33) ---------------------------------- */
uint32_t kvip_b200_update_abc(int32_t* token_to_slot, int32_t* slot_to_token,
                              const int32_t* descriptors, uint32_t groups, uint32_t rows_per_group,
                              uint32_t requests, uint32_t pool, uint32_t tokens,
                              uint32_t slots, uint32_t history, uint32_t tail, void* stream);

/* ---- Appended host pages (python/kvip/cache/page_updates.py:5-62; the Triton program it
 * replaces is python/kvip/cache/_page_updates_kernel.py:8-40). One launch publishes every
 * page appended this step, over all requests and groups: addresses[index] = address,
 * valid[index] = 1, token_to_slot[clear : clear+block] = -1 when clear >= 0, and for fused
 * groups the per-token addresses fused[group][owner, page*block + lane] =
 * address + lane * bytes_per_token[group] for tokens below `history`.
 * A row whose index or clear range is out of bounds is skipped and counted in *errors. */
typedef struct KvipPagesArgs {
  const int64_t* rows;         /* [count,3]: flat page index, host address, first map entry to clear or -1 */
  int64_t* addresses;          /* [owners, groups, pages] */
  int32_t* valid;              /* [owners, groups, pages] */
  int32_t* token_to_slot;      /* flat, map_entries long */
  const int64_t* fused_table;  /* [groups,2]: device pointer of an int64 [owners, history] table, bytes per
                                  token; NULL when no group keeps per-token addresses */
  int32_t* errors;             /* [1] in/out: rows skipped; may be NULL */
  uint64_t map_entries;
  uint32_t count, owners, groups, pages;
  uint32_t block, history, reserved0, reserved1;
} KvipPagesArgs;
uint32_t kvip_b200_publish_pages(const KvipPagesArgs* args, void* stream);

/* ---- Speculative prefetch windows ------------------------------------------------------
 * While the score kernel is still working on later key windows, rows of cold positions
 * (>= resident) whose score already beats the resident threshold are pulled from the host
 * pool (prefetch.h:577-821; budgets prefetch_budget.h:7-17: 512 rows per request and round,
 * 480 per window; predicate indexer_score.h:976-1017). The threshold of a score row is the
 * smallest score of the TopK over its resident prefix: every cold position of the final
 * TopK beats it, so the candidates are a superset of the misses. Rows are staged in a
 * separate HBM area keyed by source address, not in victim slots: the resolver, the Index
 * exchange and the slot maps behave exactly as without speculation, and the final fetch
 * copies a staged row from HBM instead of crossing the host link again. */
typedef struct KvipWindowArgs {          /* per-window bounds for windowed score launches */
  const int32_t* key_lengths;            /* [batch] */
  const int32_t* query_ends;             /* [batch*queries] */
  int32_t* window_lengths;               /* [windows, batch] out: clamp(length - first_w, 0, last_w - first_w) */
  int32_t* window_ends;                  /* [windows, batch*queries] out, same clamp of the causal bound */
  int32_t* staged_count;                 /* [batch] out: 0 */
  int32_t* staged_rows;                  /* [batch] out: 0 */
  int32_t* staged_hits;                  /* [batch] out: 0, or NULL */
  uint32_t batch, queries, windows, reserved0;
  uint32_t first[9];                     /* window w covers positions [first[w], first[w+1]); windows <= 8 */
  uint32_t reserved1;
} KvipWindowArgs;
uint32_t kvip_b200_window_bounds(const KvipWindowArgs* args, void* stream);

typedef struct KvipThresholdArgs {
  const int32_t* prefix_topk;            /* [rows, 2048] TopK over the resident prefix */
  const float* prefix_scores;            /* [rows, 2048] their scores */
  uint32_t* thresholds;                  /* [rows] out: smallest selected key (order-preserving u32 image of the
                                            score); 0 while the prefix holds fewer than 2048 valid positions */
  uint32_t rows, reserved0;
} KvipThresholdArgs;
uint32_t kvip_b200_resident_threshold(const KvipThresholdArgs* args, void* stream);

typedef struct KvipSpeculateArgs {
  const float* scores;                   /* [batch*queries, scoreStride] */
  const uint32_t* thresholds;            /* [batch*queries] keys from kvip_b200_resident_threshold */
  const int32_t* key_lengths;            /* [batch] */
  const int32_t* query_ends;             /* [batch*queries] */
  const int32_t* row_owners;             /* [batch] or NULL */
  const int64_t* addresses;              /* [owners, address_stride] source address of each Index position */
  const uint8_t* source_base;            /* device-visible base of the host pool */
  int64_t* staged_sources;               /* [batch, capacity] in/out */
  int32_t* staged_count;                 /* [batch] in/out: candidates listed so far (clamped to the limit) */
  int32_t* staged_rows;                  /* [batch] in/out: rows complete in the staging area */
  uint8_t* staging;                      /* [batch, capacity, tokenBytes] */
  uint64_t source_bytes;
  uint32_t batch, queries, scoreStride, address_stride;
  uint32_t first, last;                  /* cold window of positions, first >= resident */
  uint32_t capacity;                     /* rows per request and round (<= 512) */
  uint32_t limit;                        /* rows per request listed once this window is done (<= capacity) */
  uint32_t tokenBytes, reserved0;
} KvipSpeculateArgs;
/* Two launches: list the window's candidates, then copy their rows into the staging area. */
uint32_t kvip_b200_speculate_window(const KvipSpeculateArgs* args, void* stream);

/* ---- LIDU: the serial-chain slot resolver -------------------------------------------
 * Same 24 arguments, in the same order, as
 * nanovllm_dsa::lidu_fused_batch_get_prepare_mtp_out
 * (csrc/operators/lidu/torch_extension/csrc/lidu_fused_batch_get_prepare_mtp_ops.cpp:195-270,
 * 385-398), tensors replaced by pointers plus the sizes the checks need. */
typedef struct KvipLiduArgs {
  const int32_t* topk_indices;            /* [T,1,2048] */
  const int32_t* actual_seq_lengths_query;/* [B] cumulative ends */
  const int32_t* req_pool_entries;        /* [B] */
  int32_t* token_to_slot_pool;            /* [pool, source_capacity] in/out */
  int32_t* slot_to_token_pool;            /* [pool, resident_capacity] in/out */
  int32_t* eviction_cursors;              /* [pool] in/out */
  const int32_t* cache_tokens;            /* [B] resident budget per request */
  const int32_t* candidate_lens;          /* [B] */
  const int32_t* miss_slots;              /* [B,2048] */
  const int32_t* miss_slot_bitmap;        /* [B,4176] */
  const int32_t* resident_block_table;    /* [B, resident_blocks] */
  const int32_t* logical_seq_lengths;     /* [B] */
  const int32_t* profile_enabled;         /* [1] */
  int32_t* destination_slots;             /* [T,1,2048] out */
  int32_t* miss_counts;                   /* [B+1] out */
  int32_t* indices;                       /* [B*8192] out */
  int32_t* offsets;                       /* [B*8192] out */
  int32_t* output_indices;                /* [B*8192] out */
  int32_t* resident_seq_lengths;          /* [B] out */
  int64_t* profiling;                     /* [B,8,32] out */
  int64_t layer_id, num_layers, max_num_reqs, qcap;
  uint32_t packed_queries, batch, pool_size, source_capacity;
  uint32_t resident_capacity, resident_blocks, bitmap_words, reserved0;
  int32_t* scratch;                       /* [B, 8192*3 + 64] device work area */
} KvipLiduArgs;
uint32_t kvip_b200_lidu(const KvipLiduArgs* args, void* stream);
uint32_t kvip_b200_lidu_scratch_words(uint32_t batch);

/* ---- the fused forward -------------------------------------------------------------
 * Same call shape as the reference's
 *   uint32_t kvip_lifetch_streaming_forward(void* bindings, void* update, void* workspace,
 *                                           void* stream, const RuntimeShape* shape, uint32_t workers)
 * (include/api.h:7; op_host/launch.cpp:76-83). `bindings` = 16 x u64 (the 14 operator
 * arguments of python/kvip/operators/lifetch/workspace.py:105-123, then the context and the
 * workspace blob), `update` = 28 x i64 (python/kvip/operators/lifetch/index_update.py:12-24),
 * `workspace` = KvipWorkspace. The three blobs live in HOST memory (pinned or pageable): they
 * are read on the host at enqueue time and their values become kernel parameters, so a CUDA
 * graph captured around the call replays them without touching the blobs again.
 * Enqueues: round init -> LI score -> TopK -> resolve -> fetch -> exchange (-> gather). */
typedef struct KvipContext {          /* reference: rotating::Context, include/context.h:36-52 */
  uint64_t locations, lru_slots, reserved_hot, changes, change_slots, change_count;
  uint64_t query_ends, fetch_sources, fetch_destinations, hot_valid, row_owners;
  uint64_t token_addresses, address_stride, output_stride, tail_bounds, row_status;
  uint64_t query_counts, pool, source_base, source_bytes;
  KvipRuntimeShape shape;
  uint64_t final_posts;          /* KvipFinalPost [batch, 4] or 0 */
  uint64_t miss_mask;            /* uint32 [batch*queries, 64] or 0: needed for the overlapped commit phase */
} KvipContext;

typedef struct KvipWorkspace {        /* reference: pipeline_ab::Args, pipeline_types.h:17-22 */
  uint64_t context, keys, scales, addresses, logical_ids, hot_valid;
  uint64_t flags, events_src, events_dst, worker_status;
  uint64_t times;               /* int64 [KVIP_TIME_STAMPS] or 0; written only with KVIP_OPTION_DIAGNOSTICS */
  uint32_t history, resident, options, max_events;      /* options word at byte 96 */
  uint64_t query_bitmaps, query_errors, update_bindings;
  uint64_t dense_shadow, packed_fetch;
  uint64_t gather_out, topk_scores, li_status, topk_histogram, topk_split;
  uint64_t slots_ready_event;   /* optional cudaEvent_t recorded on the stream once the output rows are written */
  /* rows staged by kvip_b200_speculate_window (all 0 = none): the fetch takes a missing row from the
     staging area when its source address is listed there, and from the host pool otherwise */
  uint64_t staged_sources;      /* int64 [batch, staged_capacity] */
  uint64_t staged_rows;         /* int32 [batch]: rows of each request that are complete in the staging area */
  uint64_t staging;             /* uint8 [batch, staged_capacity, tokenBytes] */
  uint64_t staged_hits;         /* int32 [batch] or 0: incremented per missing row served from the staging area */
  uint32_t staged_capacity, reserved2;
  /* Overlapped commit phase (all three set, and KvipContext.miss_mask bound; 0 = everything on `stream`): the
     service outputs, the Index exchange and the gather of the entries that were hits are enqueued on `side_stream`
     while the fetch of the missing rows occupies `stream`; residency is published and the missed entries are
     gathered after both have finished. The call records `fork_event` on `stream`, makes the side stream wait for
     it, and makes `stream` wait for `join_event`, so the caller sees one ordered step (and one CUDA graph).
     No counterpart in the reference, whose forward enqueues on one stream. */
  uint64_t side_stream;         /* cudaStream_t */
  uint64_t fork_event;          /* cudaEvent_t */
  uint64_t join_event;          /* cudaEvent_t */
} KvipWorkspace;

uint32_t kvip_lifetch_streaming_forward(void* bindings, void* update, void* workspace,
                                        void* stream, const KvipRuntimeShape* shape,
                                        uint32_t workers);
/* Device timestamps of the fused forward (reference: the `times` buffer of streaming.cpp:107-108, 390-465, whose
 * per-core layout is specific to the Ascend pipeline). With KVIP_OPTION_DIAGNOSTICS the call enqueues a
 * one-thread kernel between its stages that stores the GPU's nanosecond timer: times[i] is the moment stage i
 * could start, times[i + 1] the moment it had finished, for the stages in the order below; a stage the call
 * skips repeats the previous stamp. The stamps cost a launch each: a profiling mode, off by default. */
enum { KVIP_TIME_START = 0, KVIP_TIME_LI, KVIP_TIME_TOPK, KVIP_TIME_RESOLVE, KVIP_TIME_OUTPUTS, KVIP_TIME_EXCHANGE,
       KVIP_TIME_FETCH, KVIP_TIME_GATHER, KVIP_TIME_STAMPS };
uint32_t kvip_prepare_shape(KvipRuntimeShape* shape);    /* include/api.h:9 */

/* ---- host-DDR KV pool ---------------------------------------------------------------
 * Pins `bytes` of host memory at `host` (page-aligned, owned by the caller) and maps it into the
 * device address space; *device_alias receives the pointer kernels read it through. The pool
 * and its registration must outlive every graph that was captured with it. Replaces the KVAF
 * UBmem lease (python/kvip/adapters/kvaf.py: UbmemLease; lifetch_ubmem/include/ubmem_abi.h:15-19). */
uint32_t kvip_b200_host_register(void* host, uint64_t bytes, uint64_t* device_alias);
uint32_t kvip_b200_host_unregister(void* host);
uint32_t kvip_streaming_resolver_cores(void);            /* == 3, streaming.py:41-47 */
uint32_t kvip_streaming_flag_count(void);                /* == 16 */
uint32_t kvip_b200_abi_version(void);                    /* == 3: bumped whenever an argument record of this header changes */
uint32_t kvip_b200_context_bytes(void);
uint32_t kvip_b200_workspace_bytes(void);
uint32_t kvip_b200_launch_count(void);                   /* kernels enqueued so far by this library */
const char* kvip_b200_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* KVIP_B200_H_ */
