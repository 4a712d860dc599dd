"""The allocation-free entry point (manta_b200_score_topk_static) against the regular device entry point.

Some callers cannot allocate device memory at the moment they score: the serving process gave the rest of HBM
away, its rules forbid allocation after start-up, or another stream is being captured.  For them the library
keeps one fixed scratch array in its image and offers this entry point, which uses only that array.  The test
runs it twice in a row (the array keeps the previous call's contents, so the second call proves that whatever
must start at zero is cleared) and demands the same ids and the same score bits as the regular path.  Collected
last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

import oracle
from helpers import make_rows

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_regular_path_twice():
    import torch

    from manta_b200 import native

    rt = native.Runtime(0)
    try:
        rows, cols, k = 300_000, 384, 50
        rng = np.random.default_rng(2024)
        x = make_rows(rng, rows, cols)
        codes, scales = oracle.pack_q8_rows(x)
        cands = rt.bind("q8", codes, scales, row_base=7)
        stream = torch.cuda.ExternalStream(rt.stream)
        for call_no, (nq, metric, smallest) in enumerate([(3, "cosine", False), (2, "l2_distance", True)]):
            q = make_rows(rng, nq, cols)
            with torch.cuda.stream(stream):
                d_q = torch.from_numpy(oracle.float_to_half(q).view(np.int16)).cuda()
                ref_i = torch.empty((nq, k), dtype=torch.int32, device="cuda")
                ref_s = torch.empty((nq, k), dtype=torch.float32, device="cuda")
                got_i = torch.full((nq, k), -5, dtype=torch.int32, device="cuda")
                got_s = torch.full((nq, k), -5.0, dtype=torch.float32, device="cuda")
            stream.synchronize()
            rt.score_topk_device(cands, metric, d_q, nq, k, ref_i, ref_s, smallest=smallest, sync=True)
            rt.score_topk_static(cands, metric, d_q, nq, k, got_i, got_s, smallest=smallest, sync=True)
            np.testing.assert_array_equal(got_i.cpu().numpy(), ref_i.cpu().numpy(), err_msg=f"call {call_no}")
            np.testing.assert_array_equal(got_s.cpu().numpy().view(np.uint32), ref_s.cpu().numpy().view(np.uint32),
                                          err_msg=f"call {call_no}")
            assert got_i.min().item() >= 7
            # asynchronous form: the pass's status words are checked by the next synchronisation of the runtime
            with torch.cuda.stream(stream):
                got_i.fill_(-5)
            rt.score_topk_static(cands, metric, d_q, nq, k, got_i, got_s, smallest=smallest, sync=False)
            rt.synchronize()
            np.testing.assert_array_equal(got_i.cpu().numpy(), ref_i.cpu().numpy(), err_msg=f"asynchronous call {call_no}")
        # sizes beyond the fixed scratch are refused with a clear message
        with pytest.raises(native.MantaError, match="exceed the fixed scratch"):
            rt.score_topk_static(cands, "cosine", d_q, 5, k, got_i, got_s)
        with pytest.raises(native.MantaError, match="exceeds the fixed scratch"):
            rt.score_topk_static(cands, "cosine", d_q, 1, 257, got_i, got_s)
        cands.unbind()
    finally:
        rt.close()
