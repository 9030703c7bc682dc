"""ctypes view of libkvip_b200.so: the loader and one Structure per argument struct of
include/kvip_b200.h. The product fails loudly when the CUDA library is missing."""
import ctypes
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE / "libkvip_b200.so"

u32, i32, u64, i64, vp, f32 = (ctypes.c_uint32, ctypes.c_int32, ctypes.c_uint64, ctypes.c_int64,
                               ctypes.c_void_p, ctypes.c_float)

TOPK, SLOTS, LRU_SLOTS, CHANGE_CAPACITY, BLOCK_TOKENS, MAX_QUERIES = 2048, 8192, 2048, 10240, 128, 4
OPTION_DIAGNOSTICS, OPTION_DEFERRED_FETCH = 0x80000000, 0x40000000
OPTION_LEGACY_LAYOUT, OPTION_SCHEDULING_HINTS = 0x20000000, 0x1C000000
OPTION_SELECT_ONLY, OPTION_COMMIT_ONLY, OPTION_SCORES_READY = 0x02000000, 0x01000000, 0x00800000
TOPK_SPLIT_WORDS = 20544
ERR_TOKEN_RANGE, ERR_NO_SLOT, ERR_HASH, ERR_EXCHANGE, ERR_PIPELINE, ERR_SOURCE, ERR_PEER = 1, 4, 8, 16, 32, 64, 128
PEER_HEADER_BYTES = 512
# boundaries of KvipWorkspace.times (KVIP_TIME_*)
TIME_STAGES = ("li_score", "topk", "resolve", "outputs", "exchange", "fetch", "gather")
BAD_ARGUMENT = 100000
KEY_FP8, KEY_BF16 = 0, 1
WEIGHT_BF16, WEIGHT_FP32 = 0, 1
SCORE_FP32, SCORE_BF16_AWAY = 0, 1


def _struct(name, pointer_fields, scalar_fields):
    fields = [(f, vp) for f in pointer_fields] + list(scalar_fields)
    return type(name, (ctypes.Structure,), {"_fields_": fields})


class RuntimeShape(ctypes.Structure):
    """80-byte geometry record (KvipRuntimeShape); reference: operators/lifetch/tiling.py:6-31."""

    _fields_ = [(name, u32) for name in (
        "batch", "history", "resident", "indexHeads", "smCount", "queries", "keyDtype", "weightDtype",
        "scoreMode", "pagesPerRequest", "finalWorkers", "scoreStride", "outputStride", "owners",
        "tokenBytes", "keyRows", "gatherRows", "liVariant", "reserved0", "reserved1")]

    @classmethod
    def prepare(cls, library, **fields):
        shape = cls(**fields)
        if library.kvip_prepare_shape(ctypes.byref(shape)):
            raise ValueError(f"Unsupported LIFetch runtime shape: {last_error(library)}")
        return shape


LiArgs = _struct("LiArgs", (
    "query", "keys", "weights", "query_scale", "key_scale", "key_lengths", "query_ends", "block_table",
    "scores", "status"), [(n, u32) for n in (
        "batch", "queries", "heads", "pagesPerRequest", "keyRows", "scoreStride", "keyDtype", "weightDtype",
        "scoreMode", "ctas", "stages", "withhold_tile", "wait_kilocycles", "reserved0")])

TopkArgs = _struct("TopkArgs", ("scores", "key_lengths", "query_ends", "topk", "topk_scores", "histogram"),
                   [(n, u32) for n in ("rows", "queries", "scoreStride", "base_index")] + [("split_scratch", vp)])

PackArgs = _struct("PackArgs", ("query_src", "weights_src", "scale_src", "positions_src", "gather_indices", "query_valid",
                                "query_dst", "weights_dst", "scale_dst", "position_scratch", "query_ends"),
                   [(n, u32) for n in ("rows", "tokens", "heads", "query_row_bytes", "weights_row_bytes", "reserved0")])

ColdArgs = _struct("ColdArgs", ("scores", "key_lengths", "query_ends", "prefix_topk", "prefix_scores", "threshold_keys",
                                "bitmap", "counts"),
                   [(n, u32) for n in ("rows", "queries", "scoreStride", "resident", "bitmap_words", "reserved0")])

MergeArgs = _struct("MergeArgs", ("cand_scores", "cand_index", "topk"),
                    [("rows", u32), ("shards", u32), ("shard_stride", u32), ("row_stride", u32),
                     ("peer_block", vp), ("status", vp), ("wait_ranks", u32), ("wait_kilocycles", u32)])


class PeerExchangeArgs(ctypes.Structure):
    """KvipPeerExchangeArgs: this rank's candidates and every rank's exchange block as mapped here."""

    _fields_ = [("send", vp), ("peer_block", u64 * 8), ("block_bytes", u32), ("rank", u32), ("world", u32),
                ("reserved0", u32)]

ResolveArgs = _struct("ResolveArgs", (
    "topk", "row_owners", "hot_valid", "reserved_hot", "lru_slots", "tail_bounds", "logical_ids", "addresses",
    "locations", "changes", "change_slots", "change_count", "events_src", "events_dst", "query_counts",
    "fetch_sources", "fetch_destinations", "logical_output", "slot_output", "unpack_indices", "output_valid",
    "query_ends", "row_status"), [(n, u32) for n in (
        "batch", "queries", "history", "resident", "address_stride", "outputStride", "tokenBytes", "reserved1")] + [
            ("source_bytes", u64), ("final_posts", vp), ("miss_mask", vp)])

FetchArgs = _struct("FetchArgs", (
    "source_base", "fetch_sources", "fetch_destinations", "query_counts", "row_owners", "row_status", "pool",
    "hot_valid"), [("source_bytes", u64)] + [(n, u32) for n in ("batch", "resident", "outputStride", "tokenBytes")] + [
        ("status", vp), ("defer_publication", u32), ("reserved0", u32)])

GatherArgs = _struct("GatherArgs", ("pool", "slots", "row_owners", "out"),
                     [(n, u32) for n in ("rows", "queries", "outputStride", "tokenBytes")] + [
                         ("miss_mask", vp), ("phase", u32), ("reserved0", u32)])

ExchangeArgs = _struct("ExchangeArgs", (
    "keys", "scales", "addresses", "logical_ids", "hot_valid", "events_src", "events_dst", "query_counts",
    "row_owners", "row_status", "shadow", "status"), [(n, u32) for n in (
        "batch", "queries", "history", "resident", "address_stride", "key_row_bytes", "reserved0", "reserved1")])

IngestArgs = _struct("IngestArgs", (
    "source_keys", "source_scales", "slot_mapping", "gather_indices", "query_ends", "row_owners", "keys", "scales"),
    [(n, u32) for n in ("batch", "queries", "history", "source_is_bf16")])

IngestSpanArgs = _struct("IngestSpanArgs", (
    "source_keys", "source_scales", "block_table", "slot_mapping", "positions", "spans", "keys", "scales", "errors"),
    [("source_rows", u64)] + [(n, u32) for n in ("count", "max_tokens", "owners", "history", "block", "table_rows",
                                                  "table_stride", "batch_tokens")])

LruArgs = _struct("LruArgs", ("order", "slots", "bitmap", "unique", "reserved_hot", "touched", "active"),
                  [(n, u32) for n in ("rows", "capacity", "words", "touched_stride", "resident", "reserved0",
                                      "reserved1", "reserved2")])

LiduArgs = _struct("LiduArgs", (
    "topk_indices", "actual_seq_lengths_query", "req_pool_entries", "token_to_slot_pool", "slot_to_token_pool",
    "eviction_cursors", "cache_tokens", "candidate_lens", "miss_slots", "miss_slot_bitmap", "resident_block_table",
    "logical_seq_lengths", "profile_enabled", "destination_slots", "miss_counts", "indices", "offsets",
    "output_indices", "resident_seq_lengths", "profiling"),
    [(n, i64) for n in ("layer_id", "num_layers", "max_num_reqs", "qcap")] +
    [(n, u32) for n in ("packed_queries", "batch", "pool_size", "source_capacity", "resident_capacity",
                        "resident_blocks", "bitmap_words", "reserved0")] + [("scratch", vp)])


PagesArgs = _struct("PagesArgs", ("rows", "addresses", "valid", "token_to_slot", "fused_table", "errors"),
                    [("map_entries", u64)] + [(n, u32) for n in (
                        "count", "owners", "groups", "pages", "block", "history", "reserved0", "reserved1")])


class WindowArgs(ctypes.Structure):
    _fields_ = [(n, vp) for n in ("key_lengths", "query_ends", "window_lengths", "window_ends", "staged_count",
                                  "staged_rows", "staged_hits")] + [
        (n, u32) for n in ("batch", "queries", "windows", "reserved0")] + [("first", u32 * 9), ("reserved1", u32)]


ThresholdArgs = _struct("ThresholdArgs", ("prefix_topk", "prefix_scores", "thresholds"), [("rows", u32), ("reserved0", u32)])

SpeculateArgs = _struct("SpeculateArgs", (
    "scores", "thresholds", "key_lengths", "query_ends", "row_owners", "addresses", "source_base", "staged_sources",
    "staged_count", "staged_rows", "staging"), [("source_bytes", u64)] + [(n, u32) for n in (
        "batch", "queries", "scoreStride", "address_stride", "first", "last", "capacity", "limit", "tokenBytes",
        "reserved0")])


class Context(ctypes.Structure):
    """KvipContext; reference: rotating::Context (include/context.h:36-52)."""

    _fields_ = [(n, u64) for n in (
        "locations", "lru_slots", "reserved_hot", "changes", "change_slots", "change_count", "query_ends",
        "fetch_sources", "fetch_destinations", "hot_valid", "row_owners", "token_addresses", "address_stride",
        "output_stride", "tail_bounds", "row_status", "query_counts", "pool", "source_base", "source_bytes")] + [
            ("shape", RuntimeShape), ("final_posts", u64), ("miss_mask", u64)]


class Workspace(ctypes.Structure):
    """KvipWorkspace (256 bytes); reference: pipeline_ab::Args (pipeline_types.h:17-22)."""

    _fields_ = [(n, u64) for n in (
        "context", "keys", "scales", "addresses", "logical_ids", "hot_valid", "flags", "events_src", "events_dst",
        "worker_status", "times")] + [(n, u32) for n in ("history", "resident", "options", "max_events")] + [
            (n, u64) for n in ("query_bitmaps", "query_errors", "update_bindings", "dense_shadow", "packed_fetch",
                               "gather_out", "topk_scores", "li_status", "topk_histogram", "topk_split",
                               "slots_ready_event", "staged_sources", "staged_rows", "staging", "staged_hits")] + [
            ("staged_capacity", u32), ("reserved2", u32)] + [(n, u64) for n in ("side_stream", "fork_event", "join_event")]


_STAGES = {
    "kvip_b200_li_score": LiArgs, "kvip_b200_li_score_simt": LiArgs, "kvip_b200_topk": TopkArgs,
    "kvip_b200_topk_static": TopkArgs,
    "kvip_b200_topk_merge": MergeArgs, "kvip_b200_cold_predicate": ColdArgs,
    "kvip_b200_pack_inputs": PackArgs, "kvip_b200_resolve": ResolveArgs, "kvip_b200_fetch": FetchArgs,
    "kvip_b200_gather": GatherArgs, "kvip_b200_publish_residency": FetchArgs, "kvip_b200_exchange": ExchangeArgs, "kvip_b200_ingest": IngestArgs,
    "kvip_b200_ingest_spans": IngestSpanArgs, "kvip_b200_peer_exchange": PeerExchangeArgs,
    "kvip_b200_lru_commit": LruArgs, "kvip_b200_lidu": LiduArgs, "kvip_b200_publish_pages": PagesArgs,
    "kvip_b200_window_bounds": WindowArgs, "kvip_b200_resident_threshold": ThresholdArgs,
    "kvip_b200_speculate_window": SpeculateArgs,
}
# every symbol include/kvip_b200.h declares
EXPORTS = tuple(_STAGES) + (
    "kvip_b200_update_abc", "kvip_b200_lidu_scratch_words", "kvip_lifetch_streaming_forward", "kvip_prepare_shape",
    "kvip_streaming_resolver_cores", "kvip_streaming_flag_count", "kvip_b200_abi_version",
    "kvip_b200_context_bytes", "kvip_b200_workspace_bytes", "kvip_b200_launch_count", "kvip_b200_last_error",
    "kvip_b200_host_register", "kvip_b200_host_unregister", "kvip_b200_peer_alloc", "kvip_b200_peer_open",
    "kvip_b200_peer_close", "kvip_b200_peer_free")

_library = None


def load_library(path=None):
    """Open the CUDA library and declare every entry point. Raises if it has not been built."""
    global _library
    if _library is not None and path is None:
        return _library
    target = Path(path) if path else LIBRARY_PATH
    if not target.exists():
        raise RuntimeError(
            f"{target} is missing: build it with `python -m kvip_b200.build` (nvcc, sm_100a). "
            "kvip_b200 has no CPU fallback.")
    lib = ctypes.CDLL(str(target))
    for name, struct in _STAGES.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = [ctypes.POINTER(struct), vp], u32
    lib.kvip_b200_update_abc.argtypes = [vp, vp, vp] + [u32] * 8 + [vp]
    lib.kvip_b200_update_abc.restype = u32
    lib.kvip_b200_lidu_scratch_words.argtypes, lib.kvip_b200_lidu_scratch_words.restype = [u32], u32
    lib.kvip_lifetch_streaming_forward.argtypes = [vp, vp, vp, vp, ctypes.POINTER(RuntimeShape), u32]
    lib.kvip_lifetch_streaming_forward.restype = u32
    lib.kvip_prepare_shape.argtypes, lib.kvip_prepare_shape.restype = [ctypes.POINTER(RuntimeShape)], u32
    for name in ("kvip_streaming_resolver_cores", "kvip_streaming_flag_count", "kvip_b200_abi_version",
                 "kvip_b200_context_bytes", "kvip_b200_workspace_bytes", "kvip_b200_launch_count"):
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = [], u32
    lib.kvip_b200_last_error.argtypes, lib.kvip_b200_last_error.restype = [], ctypes.c_char_p
    lib.kvip_b200_host_register.argtypes = [vp, u64, ctypes.POINTER(u64)]
    lib.kvip_b200_host_register.restype = u32
    lib.kvip_b200_host_unregister.argtypes, lib.kvip_b200_host_unregister.restype = [vp], u32
    lib.kvip_b200_peer_alloc.argtypes = [u64, ctypes.POINTER(vp), ctypes.c_char_p]
    lib.kvip_b200_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.kvip_b200_peer_close.argtypes = lib.kvip_b200_peer_free.argtypes = [vp]
    for name in ("kvip_b200_peer_alloc", "kvip_b200_peer_open", "kvip_b200_peer_close", "kvip_b200_peer_free"):
        getattr(lib, name).restype = u32
    if path is None:
        _library = lib
    return lib


def last_error(library=None):
    lib = library or load_library()
    return lib.kvip_b200_last_error().decode(errors="replace")


def check(code, what, library=None):
    """Map the C return convention to the reference's Python errors (ValueError for contract
    violations, RuntimeError for a failed launch; operators/lifetch/streaming.py:129-131)."""
    if code == 0:
        return
    message = f"{what} failed: {code} ({last_error(library)})"
    if code == BAD_ARGUMENT:
        raise ValueError(message)
    raise RuntimeError(message)
