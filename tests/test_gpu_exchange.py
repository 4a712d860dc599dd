"""Exchange of per-shard top-k lists over peer memory + merge (manta_b200_topk_exchange_merge_device).

On one GPU the exchange runs with world = 1 (the rank stores into its own inbox); with two or more GPUs a
two-process run shards a candidate set and compares the merged result of both ranks with the unsharded pass."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import make_rows, pack

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_exchange_equals_direct_pass():
    import torch

    from manta_b200 import native, sharding

    rt = native.Runtime(0)
    rng = np.random.default_rng(21)
    data, scales, _ = pack("q8", make_rows(rng, 30000, 128))
    cands = rt.bind("q8", data, scales)
    q = make_rows(rng, 5, 128)
    k = 20
    want_ids, want_sc = rt.score_topk(cands, "cosine", q, k)
    stream = torch.cuda.ExternalStream(rt.stream)
    with torch.cuda.stream(stream):
        dq = torch.from_numpy(q.astype(np.float16)).cuda()
        _, d_ids, d_sc = sharding.new_pair(5, k, "cuda")
        o_ids = torch.empty((5, k), dtype=torch.int32, device="cuda")
        o_sc = torch.empty((5, k), dtype=torch.float32, device="cuda")
    stream.synchronize()
    ex = sharding.PeerExchange(rt, None, 8, 32)
    for _ in range(3):  # both parities and a reused slot
        rt.score_topk_device(cands, "cosine", dq, 5, k, d_ids, d_sc, sync=False)
        ex.merge(d_ids, d_sc, 5, k, o_ids, o_sc, sync=True)
        np.testing.assert_array_equal(o_ids.cpu().numpy(), want_ids)
        np.testing.assert_array_equal(o_sc.cpu().numpy(), want_sc)
    for _ in range(3):  # the fused step: the shard's selection kernel stores into the inbox itself
        o_ids.zero_()
        ex.score_topk_merge(cands, "cosine", dq, 5, k, o_ids, o_sc, sync=True)
        np.testing.assert_array_equal(o_ids.cpu().numpy(), want_ids)
        np.testing.assert_array_equal(o_sc.cpu().numpy(), want_sc)
    with pytest.raises(native.MantaError, match="exceeds the exchange"):
        ex.merge(d_ids, d_sc, 9, k, o_ids, o_sc, sync=True)
    ex.close()
    cands.unbind()
    rt.close()


def test_missing_list_runs_into_the_wait_limit_and_the_runtime_stays_usable():
    """A bounded device wait running out, made on the host: two ranks' exchanges live in this process on one GPU, only
    rank 0 ever pushes, so the merge of rank 0 waits for a list nothing will write.  With a limit of a few
    milliseconds the selection kernel gives up, raises its time-out flag and returns; the call reports it, and the
    same runtime then serves an ordinary pass.  Nothing faults and no kernel waits on another kernel."""
    import torch

    from manta_b200 import native, sharding

    rt = native.Runtime(0)
    rng = np.random.default_rng(33)
    data, scales, _ = pack("q8", make_rows(rng, 20000, 64))
    cands = rt.bind("q8", data, scales)
    q = make_rows(rng, 2, 64)
    k = 8
    want_ids, want_sc = rt.score_topk(cands, "cosine", q, k)
    stream = torch.cuda.ExternalStream(rt.stream)
    with torch.cuda.stream(stream):
        dq = torch.from_numpy(q.astype(np.float16)).cuda()
        _, d_ids, d_sc = sharding.new_pair(2, k, "cuda")
        o_ids = torch.empty((2, k), dtype=torch.int32, device="cuda")
        o_sc = torch.empty((2, k), dtype=torch.float32, device="cuda")
    stream.synchronize()
    ex0, _ = rt.exchange_create(2, 0, 4, 16)
    ex1, _ = rt.exchange_create(2, 1, 4, 16)
    rt.exchange_connect_local(ex0, [ex0, ex1])
    rt.exchange_connect_local(ex1, [ex0, ex1])
    rt.exchange_set_wait_limit(ex0, 25_000)  # 25,000 naps of 200 ns: about 5 ms
    try:
        # synchronous form: the call itself fails
        with pytest.raises(native.MantaError, match="did not arrive"):
            rt.score_topk_exchange_device(ex0, cands, "cosine", dq, 2, k, o_ids, o_sc, sync=True)
        ids, sc = rt.score_topk(cands, "cosine", q, k)
        np.testing.assert_array_equal(ids, want_ids)
        np.testing.assert_array_equal(sc, want_sc)
        # two-call form, asynchronous: the next synchronisation reports it
        rt.score_topk_device(cands, "cosine", dq, 2, k, d_ids, d_sc, sync=False)
        rt.topk_exchange_merge_device(ex0, d_ids, d_sc, 2, k, o_ids, o_sc, sync=False)
        with pytest.raises(native.MantaError, match="did not arrive"):
            rt.synchronize()
        rt.synchronize()  # the report is delivered once
        ids, sc = rt.score_topk(cands, "cosine", q, k)
        np.testing.assert_array_equal(ids, want_ids)
        np.testing.assert_array_equal(sc, want_sc)
        with pytest.raises(native.MantaError, match="must be positive"):
            rt.exchange_set_wait_limit(ex0, 0)
    finally:
        rt.exchange_disconnect(ex0)
        rt.exchange_disconnect(ex1)
        rt.exchange_destroy(ex0)
        rt.exchange_destroy(ex1)
        cands.unbind()
        rt.close()


def test_overflowing_shard_pass_is_reported_and_redone():
    """A shard whose candidate pool overflows (rows sorted so that every row beats all earlier ones) holds an
    incomplete list.  The fused exchange step must not return it as a success: the list travels with a status word, the
    merge fails with a message that says so, and PeerExchange redoes the step with the chunked pass + two-call exchange."""
    import torch

    from helpers import f16_round
    from manta_b200 import native, sharding

    rt = native.Runtime(0)
    rows, cols, k = 900000, 128, 10
    rng = np.random.default_rng(9)
    q = make_rows(rng, 1, cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(1e-4)
    x += (np.arange(rows, dtype=np.float32) / rows)[:, None] * q[0][None, :]
    data, scales, _ = pack("f16", f16_round(x))
    cands = rt.bind("f16", data, scales)
    want_ids, want_sc = rt.score_topk(cands, "dot", q, k)   # the host-buffer call redoes the pass in chunks by itself
    stream = torch.cuda.ExternalStream(rt.stream)
    with torch.cuda.stream(stream):
        dq = torch.from_numpy(q.astype(np.float16)).cuda()
        o_ids = torch.zeros((1, k), dtype=torch.int32, device="cuda")
        o_sc = torch.zeros((1, k), dtype=torch.float32, device="cuda")
    stream.synchronize()
    ex = sharding.PeerExchange(rt, None, 2, 16)
    try:
        with pytest.raises(native.MantaError, match="candidate pool overflowed"):
            rt.score_topk_exchange_device(ex.ex, cands, "dot", dq, 1, k, o_ids, o_sc, sync=True)
        # asynchronous form: the next synchronisation reports it
        rt.score_topk_exchange_device(ex.ex, cands, "dot", dq, 1, k, o_ids, o_sc, sync=False)
        with pytest.raises(native.MantaError, match="candidate pool overflowed"):
            rt.synchronize()
        # the wrapper redoes the step in the form that cannot overflow
        before = rt.stats()["chunked_reruns"]
        ex.score_topk_merge(cands, "dot", dq, 1, k, o_ids, o_sc, sync=True)
        assert rt.stats()["chunked_reruns"] == before + 1
        np.testing.assert_array_equal(o_ids.cpu().numpy(), np.atleast_2d(want_ids))
        np.testing.assert_array_equal(o_sc.cpu().numpy(), np.atleast_2d(want_sc))
    finally:
        ex.close()
        cands.unbind()
        rt.close()


_CHILD = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["MB200_ROOT"]); sys.path.insert(0, os.path.join(os.environ["MB200_ROOT"], "tests"))
from helpers import make_rows, pack
from manta_b200 import native, sharding
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
rt = native.Runtime(rank)
rng = np.random.default_rng(5)
rows, cols, nq, k = 40000, 96, 6, 25
x = make_rows(rng, rows, cols)
q = make_rows(rng, nq, cols)
data, scales, _ = pack("q8", x)
r0, r1 = sharding.shard_bounds(rows, rank, world)
shard = rt.bind("q8", data[r0:r1], scales[r0:r1], row_base=r0)
stream = torch.cuda.ExternalStream(rt.stream)
with torch.cuda.stream(stream):
    dq = torch.from_numpy(q.astype(np.float16)).cuda()
    _, d_ids, d_sc = sharding.new_pair(nq, k, "cuda")
    o_ids = torch.empty((nq, k), dtype=torch.int32, device="cuda")
    o_sc = torch.empty((nq, k), dtype=torch.float32, device="cuda")
stream.synchronize()
ex = sharding.PeerExchange(rt, dist, nq, k)
whole = rt.bind("q8", data, scales)
want_ids, want_sc = rt.score_topk(whole, "cosine", q, k)
for step in range(4):
    rt.score_topk_device(shard, "cosine", dq, nq, k, d_ids, d_sc, sync=False)
    ex.merge(d_ids, d_sc, nq, k, o_ids, o_sc, sync=True)
    assert np.array_equal(o_ids.cpu().numpy(), want_ids), (rank, step)
    assert np.array_equal(o_sc.cpu().numpy(), want_sc), (rank, step)
for step in range(5):  # the fused step, mixed with the two-call form so that epochs and parities interleave
    o_ids.zero_()
    ex.score_topk_merge(shard, "cosine", dq, nq, k, o_ids, o_sc, sync=True)
    assert np.array_equal(o_ids.cpu().numpy(), want_ids), (rank, "fused", step)
    assert np.array_equal(o_sc.cpu().numpy(), want_sc), (rank, "fused", step)
    if step == 2:
        rt.score_topk_device(shard, "cosine", dq, nq, k, d_ids, d_sc, sync=False)
        ex.merge(d_ids, d_sc, nq, k, o_ids, o_sc, sync=True)
        assert np.array_equal(o_ids.cpu().numpy(), want_ids), (rank, "mixed")
ex.close()
shard.unbind(); whole.unbind(); rt.close()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_two_rank_exchange_matches_unsharded_pass(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, MB200_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29577", str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
