"""Python mirror of the MoE operator interface, over the C ABI (ctypes).

Class and method names follow the reference's Rust wrappers so tests read like
the reference's: ``RouterTopk.launch_batched`` (src/router_topk.rs:245-364),
``MoeGroupBuilder.launch`` (src/moe_group_builder.rs:72-259),
``RoutedExpertWeights`` (src/model_weights.rs:41-52), and a one-call layer in
the shape of ``MtpState::moe`` (het/mtp.rs:1606-1730).  torch is used only for
device memory and the current stream; every computation happens inside
``libdsx_moe.so``.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from ._build import LIB_PATH
from .config import FMT_MXFP4, MoeConfig, RouterConfig

SRC_MXFP4_HF, SRC_MXFP4_GGML, SRC_MXFP4_SB2, SRC_Q8_0_BLOCKS, SRC_Q8_0_SPLIT = range(5)
MAT_GATE, MAT_UP, MAT_DOWN = range(3)


class DsxError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"dsx error {code}: {msg}")
        self.code = code


class _RouterCfg(C.Structure):
    _fields_ = [("n_expert", C.c_int32), ("n_used", C.c_int32), ("n_group", C.c_int32), ("topk_group", C.c_int32),
                ("score_fn", C.c_int32), ("route_scale", C.c_float), ("weight_eps", C.c_float)]


class _MoeCfg(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("ffn", C.c_int32), ("shared_ffn", C.c_int32), ("max_tokens", C.c_int32),
                ("clamp", C.c_float), ("router", _RouterCfg)]


def _router_struct(r: RouterConfig) -> _RouterCfg:
    return _RouterCfg(r.n_expert, r.n_used, r.n_group, r.topk_group, r.score_fn, r.route_scale, r.weight_eps)


_lib = None


def lib() -> C.CDLL:
    """Load ``libdsx_moe.so``; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m deepstrix_b200._build` (there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.dsx_last_error.restype = C.c_char_p
        _lib.dsx_launch_count.restype = C.c_uint64
        _lib.dsx_wi_upper_bound.restype = C.c_uint32
        _lib.dsx_wi_upper_bound.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint64]
        _lib.dsx_ep_connect_local.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    return _lib


def _check(rc: int):
    if rc != 0:
        raise DsxError(rc, lib().dsx_last_error().decode())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dptr(t) -> C.c_void_p:
    return C.c_void_p(0) if t is None else C.c_void_p(t.data_ptr())


def launch_count(reset: bool = False) -> int:
    return int(lib().dsx_launch_count(1 if reset else 0))


def wi_upper_bound(members: int, groups: int, chunk: int, cap: int = 1 << 40) -> int:
    return int(lib().dsx_wi_upper_bound(members, groups, chunk, cap))


def bytes_per_expert(fmt: int, k: int, rows: int) -> int:
    out = C.c_size_t()
    _check(lib().dsx_bytes_per_expert(fmt, C.c_int64(k), C.c_int64(rows), C.byref(out)))
    return out.value


# --------------------------------------------------------------------------
class Module:
    """``Module::load_data`` / ``get_function`` / ``Function::launch_raw``
    (crates/v4flash-hip/src/module.rs:28-57,141-171): a code object loaded from bytes, kernels by name,
    launches with one pointer per argument."""

    def __init__(self, image: bytes):
        self._image = C.create_string_buffer(image, len(image))
        h = C.c_void_p()
        _check(lib().dsx_module_load_data(self._image, C.byref(h)))
        self._h = h

    def get_function(self, name: str) -> C.c_void_p:
        f = C.c_void_p()
        _check(lib().dsx_module_get_function(self._h, name.encode(), C.byref(f)))
        return f

    @staticmethod
    def launch_raw(fn, grid, block, shared_bytes: int, args: list):
        """args: ctypes values, one per kernel parameter, in order."""
        g = (C.c_uint32 * 3)(*grid)
        b = (C.c_uint32 * 3)(*block)
        ptrs = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
        _check(lib().dsx_function_launch(fn, g, b, C.c_uint32(shared_bytes), _stream(), ptrs))

    def close(self):
        if self._h:
            lib().dsx_module_unload(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def reduce_partials(partial: torch.Tensor, T: int, n_used: int, with_shared: bool, selected=None, expert_lo: int = 0, n_local: int = 0):
    """``launch_reduce_partials`` + ``VecAddInplace`` (q2_k_accumulate_matvec_par.hip:705-766, src/ffn.rs:118-151):
    slot-order f32 sum of the per-pick partial rows (+ the shared expert's row) -> bf16 [T, hidden]."""
    assert partial.dtype == torch.float32 and partial.is_contiguous()
    H = partial.shape[1]
    out = torch.empty((T, H), dtype=torch.bfloat16, device=partial.device)
    _check(lib().dsx_reduce_partials(_dptr(partial), C.c_int64(T), n_used, C.c_int64(H), 1 if with_shared else 0, _dptr(selected),
                                     expert_lo, n_local, _dptr(out), _stream()))
    return out


def stream_write_value32(addr: int, value: int):
    _check(lib().dsx_stream_write_value32(_stream(), C.c_void_p(addr), C.c_uint32(value)))


def stream_wait_value32(addr: int, value: int, flags: int = 0):
    _check(lib().dsx_stream_wait_value32(_stream(), C.c_void_p(addr), C.c_uint32(value), C.c_uint32(flags)))


# --------------------------------------------------------------------------
class ExpertSelCount:
    """``ExpertSelCount::launch`` (src/expert_sel_count.rs:34): accumulate the picks of one layer into the bank."""

    @staticmethod
    def launch(counts: torch.Tensor, selected: torch.Tensor, layer: int, n_expert: int):
        assert counts.dtype == torch.int32 and selected.dtype == torch.int32 and counts.is_contiguous() and selected.is_contiguous()
        assert counts.numel() >= (layer + 1) * n_expert
        _check(lib().dsx_expert_sel_count(_dptr(counts), _dptr(selected), layer * n_expert, n_expert, C.c_int64(selected.numel()), _stream()))


# --------------------------------------------------------------------------
class RmsNorm:
    """``RmsNorm::launch_weighted_batched`` (src/rms_norm.rs:161-205): rows of f32 -> normalised rows,
    as the bf16 input of the MoE layer and / or as f32."""

    @staticmethod
    def launch_weighted_batched(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, want_f32: bool = False, want_bf16: bool = True):
        assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and weight.is_contiguous()
        T, n = x.shape
        assert weight.numel() == n
        o32 = torch.empty_like(x) if want_f32 else None
        o16 = torch.empty((T, n), dtype=torch.bfloat16, device=x.device) if want_bf16 else None
        _check(lib().dsx_rms_norm_rows(_dptr(x), _dptr(weight), C.c_int64(T), C.c_int64(n), C.c_float(eps), _dptr(o32), _dptr(o16), _stream()))
        return o32, o16


class HcPost:
    """``hc_post_batched`` (src/head.rs:267-372): mixes the layer's output into the residual streams."""

    @staticmethod
    def launch_batched(block_out: torch.Tensor, residual_hc: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
        T, n_hc, n = residual_hc.shape
        assert block_out.shape == (T, n) and block_out.dtype in (torch.bfloat16, torch.float32) and block_out.is_contiguous()
        assert residual_hc.dtype == torch.float32 and residual_hc.is_contiguous()
        assert post.shape == (T, n_hc) and comb.numel() == T * n_hc * n_hc and post.is_contiguous() and comb.is_contiguous()
        out = torch.empty_like(residual_hc)
        _check(lib().dsx_hc_post(_dptr(block_out), 1 if block_out.dtype == torch.bfloat16 else 0, _dptr(residual_hc), _dptr(post), _dptr(comb),
                                 C.c_int64(T), C.c_int64(n), n_hc, _dptr(out), _stream()))
        return out


class Q8KQuantize:
    """``Q8KQuantize::launch`` (src/q8_k.rs:33-104): f32 rows -> 292-byte block_q8_K records."""

    BLOCK, BLOCK_BYTES = 256, 292

    @staticmethod
    def launch(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        assert x.dtype == torch.float32 and x.is_contiguous() and x.numel() % Q8KQuantize.BLOCK == 0
        nb = x.numel() // Q8KQuantize.BLOCK
        if out is None:
            out = torch.empty((nb * Q8KQuantize.BLOCK_BYTES,), dtype=torch.uint8, device=x.device)
        assert out.dtype == torch.uint8 and out.is_contiguous() and out.numel() >= nb * Q8KQuantize.BLOCK_BYTES
        _check(lib().dsx_q8_k_quantize(_dptr(x), C.c_int64(nb), _dptr(out), _stream()))
        return out


class SwigluClampWeighted:
    """``SwigluClampWeighted::launch`` (src/ffn.rs:91-114): mid = silu(min(gate, c)) * clamp(up) * expert_w[e]."""

    @staticmethod
    def launch(gate: torch.Tensor, up: torch.Tensor, expert_w: torch.Tensor, clamp: float, mid: torch.Tensor | None = None) -> torch.Tensor:
        n, ff = gate.shape
        assert up.shape == (n, ff) and expert_w.numel() == n
        assert all(t.dtype == torch.float32 and t.is_contiguous() for t in (gate, up, expert_w))
        if mid is None:
            mid = torch.empty_like(gate)
        _check(lib().dsx_swiglu_clamp_weighted(_dptr(mid), _dptr(gate), _dptr(up), _dptr(expert_w), C.c_float(clamp), C.c_int64(ff),
                                               C.c_int64(n), _stream()))
        return mid


class VecAddInplace:
    """``VecAddInplace`` (src/ffn.rs:118-177): ``out += rhs`` and the indexed gather ``out[i] = src[idx[i]]``."""

    @staticmethod
    def launch(out: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
        assert out.dtype == rhs.dtype == torch.float32 and out.is_contiguous() and rhs.is_contiguous() and out.numel() == rhs.numel()
        _check(lib().dsx_vec_add_inplace(_dptr(out), _dptr(rhs), C.c_int64(out.numel()), _stream()))
        return out

    @staticmethod
    def launch_gather(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        assert src.dtype == torch.float32 and idx.dtype == torch.int32 and src.is_contiguous() and idx.is_contiguous()
        out = torch.empty((idx.numel(),), dtype=torch.float32, device=src.device)
        _check(lib().dsx_gather_f32(_dptr(out), _dptr(src), _dptr(idx), C.c_int64(idx.numel()), _stream()))
        return out


# --------------------------------------------------------------------------
class RoutedExpertWeights:
    """Expert store: n_slots experts (gate, up, down) resident in HBM in the
    library's tile layout."""

    def __init__(self, fmt: int, n_slots: int, hidden: int, ffn: int, _handle=None, decode_only: bool = False):
        """decode_only: keep only the decode kernels' tile layout (an MXFP4 store otherwise also holds the
        K-major planes of the block-scaled tensor-core kernel, twice the bytes)."""
        self.fmt, self.n_slots, self.hidden, self.ffn = fmt, n_slots, hidden, ffn
        if _handle is None:
            h = C.c_void_p()
            _check(lib().dsx_expert_store_create_ex(C.byref(h), fmt, n_slots, C.c_int64(hidden), C.c_int64(ffn), C.c_uint32(1 if decode_only else 0)))
            _handle = h
        self._h = _handle

    def close(self):
        if self._h:
            lib().dsx_expert_store_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def device_bytes(self) -> int:
        out = C.c_size_t()
        _check(lib().dsx_expert_store_info(self._h, None, None, None, None, C.byref(out)))
        return out.value

    def load(self, which: int, layout: int, q, s=None, slot: int = -1):
        """Repack matrix `which` of `slot` (-1: all slots, sources back to back)
        from host numpy arrays or CUDA tensors."""
        on_dev = isinstance(q, torch.Tensor)
        if on_dev:
            assert q.is_cuda and q.is_contiguous()
            qp, sp = _dptr(q), _dptr(s)
        else:
            q = np.ascontiguousarray(q)
            s = None if s is None else np.ascontiguousarray(s)
            qp = C.c_void_p(q.ctypes.data)
            sp = C.c_void_p(0 if s is None else s.ctypes.data)
        _check(lib().dsx_expert_store_load(self._h, slot, which, layout, qp, sp, 1 if on_dev else 0, _stream()))

    def unpack(self, slot: int, which: int):
        """Inverse repack -> (q, s) CUDA uint8 tensors in HF (MXFP4) / split (Q8_0) layout."""
        rows, k = (self.hidden, self.ffn) if which == MAT_DOWN else (self.ffn, self.hidden)
        if self.fmt == FMT_MXFP4:
            q = torch.empty((rows, k // 2), dtype=torch.uint8, device="cuda")
            s = torch.empty((rows, k // 32), dtype=torch.uint8, device="cuda")
        else:
            q = torch.empty((rows, k), dtype=torch.int8, device="cuda")
            s = torch.empty((rows, k // 32), dtype=torch.float16, device="cuda")
        _check(lib().dsx_expert_store_unpack(self._h, slot, which, _dptr(q), _dptr(s), _stream()))
        return q, s

    def clone(self) -> "RoutedExpertWeights":
        h = C.c_void_p()
        _check(lib().dsx_expert_store_clone(self._h, C.byref(h), _stream()))
        return RoutedExpertWeights(self.fmt, self.n_slots, self.hidden, self.ffn, _handle=h)

    @classmethod
    def from_host(cls, fmt: int, hidden: int, ffn: int, gate, up, down, decode_only: bool = False) -> "RoutedExpertWeights":
        """gate/up/down: (q, s) numpy pairs in the canonical host layout
        (HF for MXFP4, split for Q8_0), leading dimension = slots."""
        n = gate[0].shape[0]
        st = cls(fmt, n, hidden, ffn, decode_only=decode_only)
        layout = SRC_MXFP4_HF if fmt == FMT_MXFP4 else SRC_Q8_0_SPLIT
        st.load(MAT_GATE, layout, gate[0], gate[1])
        st.load(MAT_UP, layout, up[0], up[1])
        st.load(MAT_DOWN, layout, down[0], down[1])
        return st


# --------------------------------------------------------------------------
class RouterTopk:
    """Router selection kernel wrapper."""

    def __init__(self, cfg: RouterConfig):
        self.cfg = cfg

    def logits(self, x_bf16: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
        T, H = x_bf16.shape
        E = W.shape[0]
        assert x_bf16.dtype == torch.bfloat16 and W.dtype == torch.float32 and x_bf16.is_contiguous() and W.is_contiguous()
        out = torch.empty((T, E), dtype=torch.float32, device=x_bf16.device)
        _check(lib().dsx_router_logits(_dptr(x_bf16), C.c_int64(T), _dptr(W), E, C.c_int64(H), _dptr(out), _stream()))
        return out

    def launch_batched(self, logits: torch.Tensor, bias: torch.Tensor | None):
        T, E = logits.shape
        assert E == self.cfg.n_expert and logits.dtype == torch.float32 and logits.is_contiguous()
        sel = torch.empty((T, self.cfg.n_used), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, self.cfg.n_used), dtype=torch.float32, device=logits.device)
        rc = _router_struct(self.cfg)
        _check(lib().dsx_router_topk(_dptr(logits), _dptr(bias), C.c_int64(T), C.byref(rc), _dptr(sel), _dptr(w), _stream()))
        return sel, w

    def launch_batched_ex(self, logits: torch.Tensor, bias: torch.Tensor | None, n_alt: int = 0, want_range: bool = False):
        """``launch_batched`` plus the reference's extras (src/router_topk.rs:245-364): the n_alt next-ranked
        experts per token with their weights, and the selection-score range.  Returns
        (selected, weights, alts, alt_weights, score_range); the last three are None when not asked for."""
        T, E = logits.shape
        assert E == self.cfg.n_expert and logits.dtype == torch.float32 and logits.is_contiguous()
        dev = logits.device
        sel = torch.empty((T, self.cfg.n_used), dtype=torch.int32, device=dev)
        w = torch.empty((T, self.cfg.n_used), dtype=torch.float32, device=dev)
        alts = torch.empty((T, n_alt), dtype=torch.int32, device=dev) if n_alt else None
        alt_w = torch.empty((T, n_alt), dtype=torch.float32, device=dev) if n_alt else None
        rng = torch.empty((T,), dtype=torch.float32, device=dev) if want_range else None
        rc = _router_struct(self.cfg)
        _check(lib().dsx_router_topk_ex(_dptr(logits), _dptr(bias), C.c_int64(T), C.byref(rc), _dptr(sel), _dptr(w), n_alt,
                                        _dptr(alts), _dptr(alt_w), _dptr(rng), _stream()))
        return sel, w, alts, alt_w, rng

    def launch_batched_prior(self, logits: torch.Tensor, bias: torch.Tensor | None, prior: torch.Tensor, n_protect: int, n_alt: int = 0,
                             prior_dry: bool = False):
        """The cache-prior form of ``launch_batched_ex`` (router_topk_par.hip:82-99,173-210).
        Returns (selected, weights, alts, alt_weights, orig_sel)."""
        T, E = logits.shape
        assert E == self.cfg.n_expert and logits.dtype == torch.float32 and logits.is_contiguous()
        assert prior.dtype == torch.float32 and prior.numel() == E and prior.is_contiguous()
        dev = logits.device
        sel = torch.empty((T, self.cfg.n_used), dtype=torch.int32, device=dev)
        w = torch.empty((T, self.cfg.n_used), dtype=torch.float32, device=dev)
        alts = torch.empty((T, n_alt), dtype=torch.int32, device=dev) if n_alt else None
        alt_w = torch.empty((T, n_alt), dtype=torch.float32, device=dev) if n_alt else None
        orig = torch.empty((T, self.cfg.n_used), dtype=torch.int32, device=dev)
        rc = _router_struct(self.cfg)
        _check(lib().dsx_router_topk_prior(_dptr(logits), _dptr(bias), C.c_int64(T), C.byref(rc), _dptr(sel), _dptr(w), n_alt, _dptr(alts),
                                           _dptr(alt_w), C.c_void_p(0), _dptr(prior), n_protect, 1 if prior_dry else 0, _dptr(orig), _stream()))
        return sel, w, alts, alt_w, orig


class MoeGroupBuilder:
    """Histogram / offsets / stable permutation / work items."""

    @staticmethod
    def launch_static(selected: torch.Tensor, n_expert: int, chunk: int = 32, with_work_items: bool = True):
        """Same result as :meth:`launch` through the entry point that never allocates
        device memory (the library's built-in 128 KiB scratch; at most 131072 picks).
        The output tensors are still the caller's; only the kernel's temporary moved."""
        return MoeGroupBuilder.launch(selected, n_expert, chunk, with_work_items, _entry="dsx_moe_group_build_static")

    @staticmethod
    def launch(selected: torch.Tensor, n_expert: int, chunk: int = 32, with_work_items: bool = True,
               _entry: str = "dsx_moe_group_build"):
        T, k = selected.shape
        assert selected.dtype == torch.int32 and selected.is_contiguous()
        dev = selected.device
        hist = torch.empty(n_expert, dtype=torch.int32, device=dev)
        offsets = torch.empty(n_expert + 1, dtype=torch.int32, device=dev)
        perm = torch.full((max(T * k, 1),), -1, dtype=torch.int32, device=dev)
        items = n_items = None
        if with_work_items:
            cap = wi_upper_bound(T * k, n_expert, chunk)
            items = torch.full((max(cap, 1),), -1, dtype=torch.int32, device=dev)
            n_items = torch.zeros(1, dtype=torch.int32, device=dev)
        _check(getattr(lib(), _entry)(_dptr(selected), C.c_int64(T), k, n_expert, chunk, _dptr(hist), _dptr(offsets),
                                      _dptr(perm), _dptr(items), _dptr(n_items), _stream()))
        return hist, offsets, perm, items, n_items


# --------------------------------------------------------------------------
class MoeLayer:
    """One MoE layer: router weights + routed store + shared store + workspace."""

    def __init__(self, cfg: MoeConfig, routed: RoutedExpertWeights, shared: RoutedExpertWeights | None,
                 router_w: torch.Tensor, router_bias: torch.Tensor | None, max_tokens: int = 64):
        assert router_w.is_cuda and router_w.dtype == torch.float32 and router_w.is_contiguous()
        self.cfg, self.max_tokens = cfg, max_tokens
        self._keep = (routed, shared, router_w, router_bias)
        mc = _MoeCfg(cfg.hidden, cfg.ffn, cfg.shared_ffn if shared is not None else 0, max_tokens, cfg.clamp,
                     _router_struct(cfg.router))
        h = C.c_void_p()
        _check(lib().dsx_moe_layer_create(C.byref(h), C.byref(mc), routed._h, shared._h if shared is not None else None,
                                          _dptr(router_w), _dptr(router_bias)))
        self._h = h

    def close(self):
        if self._h:
            lib().dsx_moe_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_weights(self, routed, shared, router_w, router_bias):
        _check(lib().dsx_moe_layer_set_weights(self._h, routed._h, shared._h if shared is not None else None,
                                               _dptr(router_w), _dptr(router_bias)))
        self._keep = (routed, shared, router_w, router_bias)

    def forward(self, x: torch.Tensor, logits: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        _check(lib().dsx_moe_layer_forward(self._h, _dptr(x), C.c_int64(x.shape[0]), _dptr(out), _dptr(logits), _stream()))
        return out

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """x_host/out_host: CPU bf16 tensors (pinned for speed).  Synchronous."""
        assert not x_host.is_cuda and x_host.dtype == torch.bfloat16 and x_host.is_contiguous()
        _check(lib().dsx_moe_layer_forward_host(self._h, C.c_void_p(x_host.data_ptr()), C.c_int64(x_host.shape[0]),
                                                C.c_void_p(out_host.data_ptr()), _stream()))
        return out_host

    def forward_picks(self, x, selected, weights, expert_lo: int = 0, with_shared: bool = True, out=None):
        assert selected.dtype == torch.int32 and weights.dtype == torch.float32
        if out is None:
            out = torch.empty_like(x)
        _check(lib().dsx_moe_layer_forward_picks(self._h, _dptr(x), C.c_int64(x.shape[0]), _dptr(selected), _dptr(weights),
                                                 expert_lo, 1 if with_shared else 0, _dptr(out), _stream()))
        return out

    def forward_picks_to(self, x, selected, weights, out_rows, expert_lo: int = 0, with_shared: bool = True):
        """forward_picks whose result rows are stored through ``out_rows`` (int64 CUDA tensor of T row addresses, 0 = the row is
        wanted nowhere) instead of into one buffer -- an expert-parallel owner passes ``PeerMemoryComm.back_rows()`` and its
        partial rows land in their source ranks' memory as they are produced."""
        assert selected.dtype == torch.int32 and weights.dtype == torch.float32 and out_rows.dtype == torch.int64 and out_rows.is_cuda
        assert out_rows.numel() >= x.shape[0]
        _check(lib().dsx_moe_layer_forward_picks_to(self._h, _dptr(x), C.c_int64(x.shape[0]), _dptr(selected), _dptr(weights),
                                                    expert_lo, 1 if with_shared else 0, _dptr(out_rows), _stream()))

    def forward_remap(self, x, selected, weights, remap, with_shared: bool = True, out=None):
        """Owner-side forward with the reference's ownership table (het/weights.rs:1357-1381): remap int32 [n_expert],
        negative entries -(slot + 1) are the experts this store holds."""
        assert selected.dtype == torch.int32 and weights.dtype == torch.float32 and remap.dtype == torch.int32 and remap.is_cuda
        if out is None:
            out = torch.empty_like(x)
        _check(lib().dsx_moe_layer_forward_remap(self._h, _dptr(x), C.c_int64(x.shape[0]), _dptr(selected), _dptr(weights), _dptr(remap),
                                                 remap.numel(), 1 if with_shared else 0, _dptr(out), _stream()))
        return out

    def routing(self, T: int):
        """Copies of the last forward's routing: dict of CPU numpy arrays."""
        ptrs = [C.c_void_p() for _ in range(6)]
        _check(lib().dsx_moe_layer_routing(self._h, *[C.byref(p) for p in ptrs]))
        E, k = self.cfg.router.n_expert, self.cfg.router.n_used
        shapes = {"logits": ((T, E), np.float32), "selected": ((T, k), np.int32), "weights": ((T, k), np.float32),
                  "hist": ((E,), np.int32), "offsets": ((E + 1,), np.int32), "perm": ((T * k,), np.int32)}
        torch.cuda.current_stream().synchronize()
        out = {}
        for (name, (shape, dt)), p in zip(shapes.items(), ptrs):
            if not p.value:
                out[name] = None
                continue
            a = np.empty(shape, dt)
            _check(lib().dsx_memcpy(C.c_void_p(a.ctypes.data), p, C.c_size_t(a.nbytes), 2))
            out[name] = a
        return out

    STAGES = ("router_logits", "router_topk", "group_build", "gate_up", "down", "combine")

    def profile(self, enable: bool = True):
        _check(lib().dsx_moe_layer_profile(self._h, 1 if enable else 0))

    def stage_ms(self) -> dict:
        """Device time of each stage of the last forward (profiling must be on)."""
        ms = (C.c_float * len(self.STAGES))()
        _check(lib().dsx_moe_layer_stage_ms(self._h, ms))
        return {n: float(v) for n, v in zip(self.STAGES, ms)}

    def check(self) -> int:
        """The layer's device-side error word (0 = clean).  Clears it."""
        w = C.c_uint32()
        rc = lib().dsx_moe_layer_check(self._h, _stream(), C.byref(w))
        if rc != -3:   # DSX_ERR_DEVICE only says that the word is non-zero
            _check(rc)
        return w.value


def build_layer_from_host(cfg: MoeConfig, weights: dict, max_tokens: int = 64, decode_only: bool = False):
    """weights: the dict of :func:`deepstrix_b200.synth.make_layer`."""
    routed = RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.ffn, weights["gate"], weights["up"], weights["down"], decode_only=decode_only)
    shared = None
    if cfg.shared_ffn:
        shared = RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.shared_ffn, weights["shared_gate"],
                                               weights["shared_up"], weights["shared_down"], decode_only=decode_only)
    rw = torch.from_numpy(weights["router_w"]).cuda()
    rb = torch.from_numpy(weights["router_bias"]).cuda() if weights.get("router_bias") is not None else None
    return MoeLayer(cfg, routed, shared, rw, rb, max_tokens=max_tokens)
