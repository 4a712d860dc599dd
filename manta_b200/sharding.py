"""Row sharding of a candidate set over ranks (one process per GPU) and the exchange of per-shard top-k lists.

Rank r owns the contiguous rows [r*N/G, (r+1)*N/G) and binds them with ``row_base`` = its first row, so the ids a
shard returns are global.  After the local fused pass every rank holds ``pair`` = int32 [2, nq, k] (ids, then the
f32 scores bit-cast); one all-gather produces [G, 2, nq, k] on every rank, which
``manta_b200_topk_merge_device`` reduces with ``list_stride = 2*nq*k``.
"""
from __future__ import annotations

import torch


def shard_bounds(rows: int, rank: int, world: int):
    """First and one-past-last global row of a rank's shard."""
    return rank * rows // world, (rank + 1) * rows // world


def new_pair(nq: int, k: int, device):
    """Buffer a rank's fused pass writes into: (pair, ids view, scores view)."""
    pair = torch.empty((2, nq, k), dtype=torch.int32, device=device)
    return pair, pair[0], pair[1].view(torch.float32)


def gather_pairs(pair: torch.Tensor, gathered: torch.Tensor, dist) -> torch.Tensor:
    """All-gathers every rank's pair into ``gathered`` [G, 2, nq, k] (same on all ranks)."""
    if dist.get_backend() == "nccl":
        dist.all_gather_into_tensor(gathered, pair)
    else:  # gloo (CPU tests) has no all_gather_into_tensor
        parts = [torch.empty_like(pair) for _ in range(dist.get_world_size())]
        dist.all_gather(parts, pair)
        gathered.copy_(torch.stack(parts))
    return gathered


def merge_args(gathered: torch.Tensor, nq: int, k: int):
    """(ids pointer tensor, scores pointer tensor, lists, list_stride) for manta_b200_topk_merge_device."""
    return gathered[0, 0], gathered[0, 1], gathered.shape[0], 2 * nq * k


class PeerExchange:
    """Per-shard lists exchanged with peer stores over NVLink and merged in the same stream-ordered chain
    (``manta_b200_topk_exchange_merge_device``) instead of an NCCL all-gather followed by a merge.  The inbox
    handles travel once, at set-up, through ``dist.all_gather_object``."""

    def __init__(self, rt, dist, nq_max: int, k_max: int):
        self.rt, self.dist = rt, dist
        self.world = dist.get_world_size() if dist is not None else 1
        self.rank = dist.get_rank() if dist is not None else 0
        self.ex, handle = rt.exchange_create(self.world, self.rank, nq_max, k_max)
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle)
            rt.exchange_connect(self.ex, handles)
            dist.barrier()  # every inbox is mapped everywhere before the first push

    @classmethod
    def try_create(cls, rt, dist, nq_max: int, k_max: int):
        """A connected exchange, or None on EVERY rank when any rank could not create or map the inboxes (no
        peer access between the GPUs, IPC handles not permitted): the ranks agree through one all-reduce."""
        import torch

        self = cls.__new__(cls)
        self.rt, self.dist, self.ex = rt, dist, None
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        ok, handle = 1, b"\0" * 64
        try:
            self.ex, handle = rt.exchange_create(self.world, self.rank, nq_max, k_max)
        except Exception:
            ok = 0
        handles = [None] * self.world
        dist.all_gather_object(handles, handle)
        if ok:
            try:
                rt.exchange_connect(self.ex, handles)
            except Exception:
                ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device="cuda" if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            # every rank is here (the all-reduce above): unmap, meet, and only then free the inboxes
            if self.ex is not None:
                rt.exchange_disconnect(self.ex)
            dist.barrier()
            if self.ex is not None:
                rt.exchange_destroy(self.ex)
            return None
        dist.barrier()
        return self

    def merge(self, d_ids, d_scores, nq: int, k: int, d_out_ids, d_out_scores, smallest: bool = False, sync: bool = False):
        self.rt.topk_exchange_merge_device(self.ex, d_ids, d_scores, nq, k, d_out_ids, d_out_scores, smallest=smallest, sync=sync)

    def score_topk_merge(self, cands, metric: str, d_queries, nq: int, k: int, d_out_ids, d_out_scores, smallest: bool = False,
                         sync: bool = False):
        """The whole sharded step: this rank's fused pass stores its lists into every inbox, then the merge.

        A shard whose candidate pool overflows (rows arriving in an order that defeats the in-scan filter) marks its list
        incomplete, and the merge fails on EVERY rank.  With ``sync`` the step is then redone here, on all ranks alike, in
        the form that cannot overflow: the chunked synchronous pass followed by the two-call exchange.  Without ``sync``
        the failure is reported by the runtime's next ``synchronize``."""
        from .native import MantaError

        try:
            self.rt.score_topk_exchange_device(self.ex, cands, metric, d_queries, nq, k, d_out_ids, d_out_scores, smallest=smallest,
                                               sync=sync)
        except MantaError as exc:
            if not sync or "candidate pool overflowed" not in str(exc):
                raise
            pair = torch.empty((2, nq, k), dtype=torch.int32, device=d_out_ids.device)
            self.rt.score_topk_device(cands, metric, d_queries, nq, k, pair[0], pair[1].view(torch.float32), smallest=smallest, sync=True)
            self.rt.topk_exchange_merge_device(self.ex, pair[0], pair[1].view(torch.float32), nq, k, d_out_ids, d_out_scores,
                                               smallest=smallest, sync=True)

    def close(self):
        """Every rank reaches the barrier and releases its inbox even when its last pass reported an error (the
        error is raised afterwards), so a failing rank cannot strand the others."""
        if self.ex is None:
            return
        pending = None
        try:
            self.rt.synchronize()
        except Exception as exc:  # reported below, after the collective part
            pending = exc
        # CUDA IPC wants every importer to unmap before the exporter frees: all ranks finish their work, unmap the
        # peers' inboxes, meet again, and only then free their own
        if self.world > 1:
            self.dist.barrier()  # no rank unmaps an inbox a peer may still store into
        try:
            self.rt.exchange_disconnect(self.ex)
        except Exception as exc:
            pending = pending or exc
        if self.world > 1:
            self.dist.barrier()  # no rank frees an inbox a peer still has mapped
        self.rt.exchange_destroy(self.ex)
        self.ex = None
        if pending is not None:
            raise pending
