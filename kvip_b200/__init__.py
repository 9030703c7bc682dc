"""kvip_b200: the DeepSeek-sparse-attention selection-and-fetch path of KVIP as CUDA for B200.

Public names are those of the reference package (python/kvip/__init__.py:7-28) and resolve lazily."""
from importlib import import_module

__all__ = ["QueryInputs", "LIFetchWorkspace", "IndexCacheStorage", "LIFetch", "SlotLRU", "bind_selectors",
           "build_libraries", "lidu", "update_abc"]
_EXPORTS = {
    "lidu": ("operators.lidu", "lidu"),
    "QueryInputs": ("inputs", "QueryInputs"),
    "LIFetchWorkspace": ("operators.lifetch", "LIFetchWorkspace"),
    "IndexCacheStorage": ("cache.index_storage", "IndexCacheStorage"),
    "LIFetch": ("operators.lifetch", "LIFetch"),
    "SlotLRU": ("cache.lru", "SlotLRU"),
    "update_abc": ("cache.abc", "update_abc"),
    "bind_selectors": ("adapters", "bind_selectors"),
    "build_libraries": ("adapters", "build_libraries"),
    # objects this build adds next to the reference's names
    "CudaBinding": ("operators.lifetch", "CudaBinding"),
    "IndexUpdate": ("operators.lifetch", "IndexUpdate"),
    "HostKVPool": ("operators.lifetch", "HostKVPool"),
    "HostDecodeLoop": ("host_loop", "HostDecodeLoop"),
    "IndexSelector": ("adapters", "IndexSelector"),
    "PagedIndexer": ("adapters", "PagedIndexer"),
    "RequestPlan": ("adapters", "RequestPlan"),
    "PageUpdates": ("cache.page_updates", "PageUpdates"),  # reference: kvip.cache.page_updates.PageUpdates
    "FusedQueryInputs": ("inputs", "QueryInputs"),
    "FusedWorkspace": ("operators.lifetch", "LIFetchWorkspace"),
}


def __getattr__(name):
    if name not in _EXPORTS:
        raise AttributeError(name)
    module, symbol = _EXPORTS[name]
    return getattr(import_module(f"{__name__}.{module}"), symbol)
