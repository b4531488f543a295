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


# --------------------------------------------------------------------------
# The same step over peer memory: rows go straight into the owner's device memory (CUDA IPC
# mapping of one slab per rank), slots come from a scan on the device, and nothing in the step
# synchronises with the host.  The arithmetic (what is sent, the rank-order f32 sum) is the one
# above, so both transports give the same bits.
class _DeviceView:
    """A device pointer as a zero-copy torch tensor (through __cuda_array_interface__)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


def _as_tensor(ptr: int, shape, typestr: str, dtype=None) -> torch.Tensor:
    t = torch.as_tensor(_DeviceView(ptr, shape, typestr), device="cuda")
    return t if dtype is None else t.view(dtype)


class PeerMemoryComm:
    """One rank's end of the exchange (``dsx_ep_*`` of the C ABI)."""

    def __init__(self, world: int, rank: int, cap: int, hidden: int, n_used: int):
        import ctypes as C
        from . import moe
        self._C, self._moe = C, moe
        self.world, self.rank, self.cap, self.hidden, self.k = world, rank, cap, hidden, n_used
        h = C.c_void_p()
        moe._check(moe.lib().dsx_ep_create(world, rank, C.c_int64(cap), C.c_int64(hidden), n_used, C.byref(h)))
        self._h = h

    def export_handle(self) -> bytes:
        buf = (self._C.c_uint8 * 64)()
        self._moe._check(self._moe.lib().dsx_ep_export(self._h, buf))
        return bytes(buf)

    def connect(self, handles: list):
        blob = b"".join(handles)
        assert len(blob) == 64 * self.world
        self._moe._check(self._moe.lib().dsx_ep_connect(self._h, (self._C.c_uint8 * len(blob)).from_buffer_copy(blob)))

    def connect_local(self, ranks: list):
        arr = (self._C.c_void_p * self.world)(*[r._h for r in ranks])
        self._moe._check(self._moe.lib().dsx_ep_connect_local(self._h, arr))

    def connect_group(self, group=None):
        """Exchange the slab handles over the process group (ranks are processes on one node)."""
        handles = [None] * self.world
        dist.all_gather_object(handles, self.export_handle(), group=group)
        self.connect(handles)

    def dispatch(self, x, selected, weights, n_expert: int):
        m, C = self._moe, self._C
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and selected.dtype == torch.int32 and weights.dtype == torch.float32
        assert selected.is_contiguous() and weights.is_contiguous()
        m._check(m.lib().dsx_ep_dispatch(self._h, m._dptr(x), m._dptr(selected), m._dptr(weights), C.c_int64(x.shape[0]), n_expert, m._stream()))

    def barrier(self):
        self._moe._check(self._moe.lib().dsx_ep_barrier(self._h, self._moe._stream()))

    def prepare(self):
        """(rows [world*cap, hidden] bf16, picks [world*cap, k] int32, weights [world*cap, k] f32), views of library memory."""
        m, C = self._moe, self._C
        px, ps, pw, n = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_int64()
        m._check(m.lib().dsx_ep_prepare(self._h, C.byref(px), C.byref(ps), C.byref(pw), C.byref(n), m._stream()))
        slots = n.value
        rows = _as_tensor(px.value, (slots, self.hidden), "<i2", torch.bfloat16)
        return rows, _as_tensor(ps.value, (slots, self.k), "<i4"), _as_tensor(pw.value, (slots, self.k), "<f4")

    def back_rows(self) -> torch.Tensor:
        """After prepare(): int64 [world*cap] addresses, entry i = where slot i's partial row belongs in its source rank's slab
        (0 for an unused slot); for ``MoeLayer.forward_picks_to``."""
        p = self._C.c_void_p()
        self._moe._check(self._moe.lib().dsx_ep_back_rows(self._h, self._C.byref(p)))
        return _as_tensor(p.value, (self.world * self.cap,), "<i8")

    def give_back(self, part):
        assert part.dtype == torch.bfloat16 and part.is_contiguous() and part.shape == (self.world * self.cap, self.hidden)
        self._moe._check(self._moe.lib().dsx_ep_give_back(self._h, self._moe._dptr(part), self._moe._stream()))

    def sum(self, shared, T: int, out=None):
        m, C = self._moe, self._C
        if out is None:
            out = torch.empty((T, self.hidden), dtype=torch.bfloat16, device="cuda")
        m._check(m.lib().dsx_ep_sum(self._h, m._dptr(shared), C.c_int64(T), m._dptr(out), m._stream()))
        return out

    def counts(self) -> torch.Tensor:
        p = self._C.c_void_p()
        self._moe._check(self._moe.lib().dsx_ep_counts(self._h, self._C.byref(p)))
        return _as_tensor(p.value, (self.world,), "<i4")

    def set_barrier_polls(self, polls: int):
        """Polls (>= 100 ns each) a barrier waits for its peers before it gives up with error bit 1."""
        self._moe._check(self._moe.lib().dsx_ep_set_barrier_polls(self._h, self._C.c_uint32(polls)))

    def check(self) -> int:
        """The exchange kernels' error word (0 = clean; bit 1 = a barrier gave up waiting).  Clears it."""
        w = self._C.c_uint32()
        rc = self._moe.lib().dsx_ep_check(self._h, self._moe._stream(), self._C.byref(w))
        if rc != -3:   # DSX_ERR_DEVICE only says that the word is non-zero
            self._moe._check(rc)
        return int(w.value)

    def close(self):
        if self._h:
            self._moe.lib().dsx_ep_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ExpertParallelPeerMemory:
    """ExpertParallelMoe's step with the peer-memory transport (GPU ranks of one node).

    local_compute(rows, selected, weights) must accept world*cap rows whose unused slots carry picks of -1
    (``MoeLayer.forward_picks`` does) and return one bf16 row per slot.  shared_compute runs on a side
    stream at the same time as local_compute: the two callables must not share a ``MoeLayer`` (a layer's
    workspace serves one call at a time)."""

    def __init__(self, n_expert: int, comm: PeerMemoryComm, local_compute: Callable, shared_compute: Callable = None,
                 local_compute_to: Callable = None):
        """local_compute_to(rows, selected, weights, out_rows), when given, replaces local_compute + give_back: the owner's layer
        stores every partial row straight into its source rank's slab (``MoeLayer.forward_picks_to``)."""
        self.n_expert, self.comm = n_expert, comm
        self.local_compute, self.shared_compute, self.local_compute_to = local_compute, shared_compute, local_compute_to
        self._side = None
        self.profile = False
        self._events = []
        self.last_stats = {}

    _mark = ExpertParallelMoe._mark
    phase_ms = ExpertParallelMoe.phase_ms

    def forward(self, x: torch.Tensor, selected: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        c = self.comm
        T = x.shape[0]
        self._mark("start")
        c.dispatch(x, selected, weights, self.n_expert)
        sh = None
        if self.shared_compute is not None:   # beside the exchange, on a side stream
            if self._side is None:
                self._side = torch.cuda.Stream()
            main = torch.cuda.current_stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                sh = self.shared_compute(x)
                sh.record_stream(main)
        c.barrier()
        self._mark("dispatch_and_barrier")
        rows, sel, w = c.prepare()
        if self.local_compute_to is not None:
            self.local_compute_to(rows, sel, w, c.back_rows())   # the result rows cross NVLink as they are produced
            self._mark("owned_experts")
        else:
            part = self.local_compute(rows, sel, w)
            self._mark("owned_experts")
            c.give_back(part)
        c.barrier()
        if sh is not None:
            torch.cuda.current_stream().wait_stream(self._side)
        out = c.sum(sh, T)
        self._mark("give_back_barrier_and_sum")
        return out
