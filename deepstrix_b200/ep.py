"""Expert parallelism: experts sharded over the ranks of one node, token dispatch
and combine as all-to-all exchanges.

Semantics follow the reference's remote-expert protocol
(docs/v41/REMOTE_EXPERTS.md:163-164,196-229; het/remote_experts.rs:7428-7442): a
token is sent ONCE to every rank that owns at least one of its picks, together
with all its picks and weights; the owner skips the picks it does not own (as
NO_PICK is skipped) and returns one weighted partial-sum row per received
token; the sender adds the partials in rank order to its local shared-expert
output.  The exchange is per-peer send/recv inside one batch (NCCL groups the
calls; gloo runs the same code on CPU for the tests).

This module is plumbing: `local_compute` is the C-ABI operator
(`MoeLayer.forward_picks`) on a GPU, or any callable with the same contract.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def owner_of(selected: torch.Tensor, experts_per_rank: int) -> torch.Tensor:
    """Rank owning each pick (-1 for NO_PICK)."""
    return torch.where(selected >= 0, torch.div(selected, experts_per_rank, rounding_mode="floor"), torch.full_like(selected, -1))


def build_dispatch(selected: torch.Tensor, world: int, experts_per_rank: int):
    """For every destination rank the ascending list of local tokens with at
    least one pick owned there.  Returns (token index tensor sorted by
    (destination, token), counts per destination as a CPU list)."""
    T = selected.shape[0]
    own = owner_of(selected, experts_per_rank)                       # [T, k]
    mask = torch.zeros((T, world), dtype=torch.bool, device=selected.device)
    valid = own >= 0
    rows = torch.arange(T, device=selected.device).unsqueeze(1).expand_as(own)
    mask[rows[valid], own[valid].long()] = True
    dst, tok = torch.nonzero(mask.t(), as_tuple=True)                # sorted by destination, then token
    counts = torch.bincount(dst, minlength=world)
    return tok, counts


def _exchange(send: list, recv: list, group, rank: int):
    """send[d] goes to rank d, recv[s] is filled from rank s (same dtype/shape contract on both sides)."""
    ops = []
    for peer in range(len(send)):
        if peer == rank:
            recv[peer].copy_(send[peer])
            continue
        if recv[peer].numel():
            ops.append(dist.P2POp(dist.irecv, recv[peer], dist.get_global_rank(group, peer) if group is not None else peer, group))
        if send[peer].numel():
            ops.append(dist.P2POp(dist.isend, send[peer], dist.get_global_rank(group, peer) if group is not None else peer, group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


class ExpertParallelMoe:
    """One expert-parallel MoE layer step.

    local_compute(x_rows, selected, weights) -> partial rows  (picks outside the
        rank's expert range are skipped; no shared expert)
    shared_compute(x_rows) -> shared expert output for the rank's own tokens (or None)
    """

    def __init__(self, n_expert: int, group=None, local_compute: Callable = None, shared_compute: Callable = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert n_expert % self.world == 0, "experts must split evenly over the ranks"
        self.experts_per_rank = n_expert // self.world
        self.local_compute = local_compute
        self.shared_compute = shared_compute
        self.last_stats = {}
        self._side = None   # side stream: the shared expert runs beside the dispatch exchange
        self.profile = False  # when set, forward() brackets its phases with CUDA events (see phase_ms)
        self._events = []

    def _mark(self, name):
        if self.profile:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._events.append((name, e))

    def phase_ms(self) -> dict:
        """Device time per phase accumulated since the last call (profile mode)."""
        torch.cuda.synchronize()
        out = {}
        for (n0, e0), (n1, e1) in zip(self._events[:-1], self._events[1:]):
            if n1 != "start":
                out[n1] = out.get(n1, 0.0) + e0.elapsed_time(e1)
        self._events = []
        return out

    def forward(self, x: torch.Tensor, selected: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        W, r = self.world, self.rank
        self._mark("start")
        T, H = x.shape
        k = selected.shape[1]
        tok, counts = build_dispatch(selected, W, self.experts_per_rank)
        # counts[src][dst] everywhere (one small all-gather; the only host round trip of the step)
        all_counts = [torch.empty_like(counts) for _ in range(W)]
        dist.all_gather(all_counts, counts, group=self.group)
        cm = torch.stack(all_counts).cpu()                             # [src, dst]
        send_n = cm[r].tolist()
        recv_n = cm[:, r].tolist()
        self._mark("dispatch_lists_and_counts")
        # pack rows and (picks | weights bit-cast) per destination
        xs = x.index_select(0, tok)
        meta = torch.cat([selected.index_select(0, tok), weights.index_select(0, tok).view(torch.int32)], dim=1)
        send_x = list(torch.split(xs, send_n))
        send_m = list(torch.split(meta, send_n))
        R = int(sum(recv_n))
        rx = torch.empty((R, H), dtype=x.dtype, device=x.device)
        rm = torch.empty((R, 2 * k), dtype=torch.int32, device=x.device)
        recv_x = list(torch.split(rx, recv_n))
        recv_m = list(torch.split(rm, recv_n))
        # shared expert of the rank's own tokens: independent of the exchange, so on a GPU it runs
        # on a side stream while the rows travel (het/forward_layer.rs:50-80 overlaps the same way)
        sh = None
        if self.shared_compute is not None and x.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream()
            main = torch.cuda.current_stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                sh = self.shared_compute(x)
                sh.record_stream(main)
        _exchange(send_x, recv_x, self.group, r)
        _exchange(send_m, recv_m, self.group, r)
        if self.shared_compute is not None and not x.is_cuda:
            sh = self.shared_compute(x)
        self._mark("pack_and_dispatch_exchange")
        if sh is not None and x.is_cuda:
            torch.cuda.current_stream().wait_stream(self._side)
        self._mark("wait_shared_expert")
        out = sh.float() if sh is not None else torch.zeros((T, H), dtype=torch.float32, device=x.device)
        # owned experts on everything received
        if R:
            part = self.local_compute(rx, rm[:, :k].contiguous(), rm[:, k:].contiguous().view(torch.float32))
        else:
            part = torch.empty((0, H), dtype=x.dtype, device=x.device)
        self._mark("owned_experts")
        # combine: partial rows travel back the way the tokens came
        back = torch.empty((tok.numel(), H), dtype=x.dtype, device=x.device)
        _exchange(list(torch.split(part, recv_n)), list(torch.split(back, send_n)), self.group, r)
        # add in rank order: fixed association, every token at most once per rank
        off = 0
        for d in range(W):
            n = send_n[d]
            if n:
                out.index_add_(0, tok[off:off + n], back[off:off + n].float())
                off += n
        self._mark("combine_exchange_and_sum")
        self.last_stats = {"sent_rows": int(tok.numel()), "received_rows": R, "fanout": float(tok.numel()) / max(T, 1)}
        return out.to(x.dtype)
