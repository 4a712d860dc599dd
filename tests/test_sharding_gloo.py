"""The N>1 host path on CPU: two gloo ranks shard a candidate set, score their shards (the oracle stands in for the
device scan), exchange their [2, nq, k] lists with the same gather helper the GPU path uses, and the merged result
must equal the unsharded oracle's -- ids and scores, for largest and smallest orders."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _merge_reference(gathered: np.ndarray, k: int, smallest: bool):
    """CPU statement of the merge rule: best k of the union by (score, then lower id)."""
    lists, _, nq, _ = gathered.shape
    ids = gathered[:, 0].transpose(1, 0, 2).reshape(nq, -1)
    scores = gathered[:, 1].view(np.float32).transpose(1, 0, 2).reshape(nq, -1)
    out_i = np.empty((nq, k), np.int32)
    out_s = np.empty((nq, k), np.float32)
    for q in range(nq):
        key = scores[q] if smallest else -scores[q]
        order = np.lexsort((ids[q], key))[:k]
        out_i[q], out_s[q] = ids[q][order], scores[q][order]
    return out_i, out_s


def _worker(rank, world, port, rows, cols, nq, k, metric, smallest, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from helpers import make_rows
    from manta_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(99)  # same seed on every rank: every rank can form any shard
        x = make_rows(rng, rows, cols)
        q = make_rows(rng, nq, cols)
        r0, r1 = sharding.shard_bounds(rows, rank, world)
        ids, sc = oracle.score_topk(metric, q, x[r0:r1], k, smallest)
        pair, p_ids, p_sc = sharding.new_pair(nq, k, "cpu")
        p_ids.copy_(torch.from_numpy(ids + r0))  # row_base makes ids global
        p_sc.copy_(torch.from_numpy(sc))
        gathered = torch.empty((world, 2, nq, k), dtype=torch.int32)
        sharding.gather_pairs(pair, gathered, dist)
        g_ids, g_sc, lists, stride = sharding.merge_args(gathered, nq, k)
        assert lists == world and stride == 2 * nq * k
        assert g_sc.data_ptr() - g_ids.data_ptr() == nq * k * 4
        m_ids, m_sc = _merge_reference(gathered.numpy(), k, smallest)
        w_ids, w_sc = oracle.score_topk(metric, q, x, k, smallest)
        np.testing.assert_array_equal(m_ids, w_ids)
        np.testing.assert_array_equal(m_sc, w_sc)
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def _run(metric, smallest, k, port):
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, 5001, 64, 3, k, metric, smallest, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def test_two_rank_shard_gather_merge_cosine():
    _run("cosine", False, 10, 29621)


def test_two_rank_shard_gather_merge_l2_smallest():
    _run("l2_distance", True, 100, 29622)


def test_shard_bounds_cover_rows_exactly():
    from manta_b200 import sharding

    for rows in (0, 1, 7, 10_000_000, 100_000_001):
        for world in (1, 2, 3, 8):
            b = [sharding.shard_bounds(rows, r, world) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == rows
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            assert max(e - s for s, e in b) - min(e - s for s, e in b) <= 1


class _FakeRuntime:
    """Stands in for native.Runtime in the host logic of the peer exchange: records calls, fails on request."""

    def __init__(self, fail_create=False, fail_connect=False):
        self.fail_create, self.fail_connect = fail_create, fail_connect
        self.created = self.connected = self.destroyed = self.disconnected = 0
        self.log = []  # call order, shared with the barrier spy

    def exchange_create(self, world, rank, nq_max, k_max):
        if self.fail_create:
            raise RuntimeError("no IPC here")
        self.created += 1
        return object(), bytes([rank]) * 64

    def exchange_connect(self, ex, handles):
        if self.fail_connect:
            raise RuntimeError("cannot map a peer")
        assert len(handles) == 2 and handles[0] == bytes([0]) * 64 and handles[1] == bytes([1]) * 64
        self.connected += 1

    def exchange_disconnect(self, ex):
        self.disconnected += 1
        self.log.append("disconnect")

    def exchange_destroy(self, ex):
        self.destroyed += 1
        self.log.append("destroy")

    def synchronize(self):
        self.log.append("synchronize")


class _DistSpy:
    """torch.distributed with every barrier noted in the fake runtime's call log."""

    def __init__(self, real, log):
        self._real, self._log = real, log

    def barrier(self, *a, **kw):
        self._log.append("barrier")
        return self._real.barrier(*a, **kw)

    def __getattr__(self, name):
        return getattr(self._real, name)


def _exchange_worker(rank, world, port, scenario, ret):
    sys.path.insert(0, ROOT)
    from manta_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rt = _FakeRuntime(fail_create=(scenario == "create" and rank == 1), fail_connect=(scenario == "connect" and rank == 0))
        spy = _DistSpy(dist, rt.log)
        px = sharding.PeerExchange.try_create(rt, spy, 4, 10)
        if scenario == "ok":
            assert px is not None and rt.created == 1 and rt.connected == 1
            del rt.log[:]
            px.close()
            assert rt.destroyed == 1
            # an inbox is freed only after every rank has unmapped it: unmap, barrier, free
            assert rt.log == ["synchronize", "barrier", "disconnect", "barrier", "destroy"]
        else:
            # one rank failed: EVERY rank falls back, and a rank that had created its inbox releases it, again with a
            # barrier between the unmapping and the freeing
            assert px is None
            assert rt.destroyed == rt.created
            assert rt.log[-1 - rt.created:] == (["disconnect"] * rt.created + ["barrier"] + ["destroy"] * rt.created)[-1 - rt.created:]
            assert "barrier" in rt.log and (not rt.created or rt.log.index("disconnect") < len(rt.log) - 1 - rt.log[::-1].index("barrier") < rt.log.index("destroy"))
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def _run_exchange(scenario, port):
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_exchange_worker, args=(2, port, scenario, ret), nprocs=2, join=True)
        assert all(ret.get(r) for r in range(2))


def test_peer_exchange_setup_and_agreed_fallback():
    _run_exchange("ok", 29631)
    _run_exchange("create", 29632)
    _run_exchange("connect", 29633)
