"""Names of the reference's serving adapter that lie outside this build.

`bind_selectors` needs vLLM-Ascend policy/writer objects and `build_libraries` drives the Ascend
toolchain (reference python/kvip/adapters/vllm/binding.py:20-200, python/kvip/runtime/build.py:40-91);
both names exist so that `import kvip_b200` offers the reference's surface, and say what to use instead."""


def bind_selectors(*_args, **_kwargs):
    raise NotImplementedError(
        "bind_selectors binds vLLM-Ascend layer objects; on CUDA build the path from LIFetchWorkspace, "
        "IndexCacheStorage, CudaBinding, IndexUpdate and LIFetch (see INTEGRATION.md)")


def build_libraries(force=False):
    """Build the CUDA library in-tree and return its path (the reference built three Ascend libraries)."""
    from .build import build_library

    return {"lifetch": build_library(force=force)}
