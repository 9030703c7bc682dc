"""TopK through the entry point that allocates nothing (B200 only; collected last on purpose).

`kvip_b200_topk_static` exists for hosts that cannot hand the library a scratch buffer - a serving process
whose cache pool already owns all free HBM, a decode-loop plugin that must not allocate - so it keeps its
histogram scratch inside the library image. It must select exactly what `kvip_b200_topk` selects, call
after call, although every call finds the previous call's leftovers in the shared scratch."""
import ctypes

import numpy as np
import pytest
import torch

import oracle_c
from kvip_b200 import _lib

pytestmark = pytest.mark.gpu
TOPK = 2048


def _outputs(scores):
    return (torch.full((scores.shape[0], TOPK), -9, dtype=torch.int32, device=scores.device),
            torch.zeros((scores.shape[0], TOPK), dtype=torch.float32, device=scores.device))


def _call(entry, scores, lengths, ends, histogram=None, outputs=None):
    device = scores.device
    out, out_scores = outputs or _outputs(scores)
    args = _lib.TopkArgs(scores=scores.data_ptr(), key_lengths=lengths.data_ptr(), query_ends=ends.data_ptr(),
                         topk=out.data_ptr(), topk_scores=out_scores.data_ptr(),
                         histogram=None if histogram is None else histogram.data_ptr(), rows=scores.shape[0],
                         queries=scores.shape[0] // lengths.numel(), scoreStride=scores.shape[1], base_index=0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    code = getattr(_lib.load_library(), entry)(ctypes.byref(args), stream)
    return code, out, out_scores


def test_static_scratch_topk_matches_the_allocating_entry_point(device):
    rng = np.random.default_rng(17)
    # two calls in a row with different shapes and data: the second one meets the first one's leftovers
    cases = [
        (rng.standard_normal((12, 40960)).astype(np.float32), np.array([40960, 30000, 2049, 100, 0, 40960], np.int32), 2),
        (rng.integers(-3, 4, (5, 16384)).astype(np.float32), np.array([16384, 9000, 16384, 2048, 16000], np.int32), 1),
    ]
    for scores_np, lengths_np, queries in cases:
        scores = torch.from_numpy(scores_np).to(device)
        lengths = torch.from_numpy(lengths_np).to(device)
        ends = torch.from_numpy(np.repeat(lengths_np, queries).astype(np.int32)).to(device)
        histogram = torch.zeros((scores.shape[0], 4096), dtype=torch.int32, device=device)
        code, expected, expected_scores = _call("kvip_b200_topk", scores, lengths, ends, histogram)
        assert code == 0
        outputs = _outputs(scores)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(device)[0]
        count_before = torch.cuda.memory_stats(device)["allocation.all.allocated"]
        code, static_out, static_scores = _call("kvip_b200_topk_static", scores, lengths, ends, outputs=outputs)
        assert code == 0, _lib.last_error()
        torch.cuda.synchronize()
        # neither the driver's free memory nor torch's allocation count moved across the call
        assert torch.cuda.mem_get_info(device)[0] == free_before
        assert torch.cuda.memory_stats(device)["allocation.all.allocated"] == count_before
        assert torch.equal(static_out, expected) and torch.equal(static_scores, expected_scores)
        # and both are the oracle's selection (C restatement of the canonical order)
        assert np.array_equal(static_out.cpu().numpy(), oracle_c.topk(scores_np, lengths_np, ends.cpu().numpy()))


def test_static_scratch_topk_rejects_more_rows_than_it_holds(device):
    scores = torch.zeros((257, 4096), dtype=torch.float32, device=device)
    lengths = torch.full((257,), 4096, dtype=torch.int32, device=device)
    code, _, _ = _call("kvip_b200_topk_static", scores, lengths, lengths)
    assert code == _lib.BAD_ARGUMENT and "256" in _lib.last_error()
