"""A decode step's whole stack of layers as one resident kernel (csrc/decode_stack.cu): the plan that
turns a built model into the kernel's program of phases, and the launch.

The plan looks at the model's layers as data: it takes a layer whose arrangement is the pre-norm
block, whose norms are RMS norms, whose mixer is the attention part (head size 64 or 128, groups
of up to 16, no position encoding or one the decode kernels apply to whole heads) and whose
feed-forward is the gated SiLU part with interleaved gate/up rows, all in bfloat16.  A model with
any other layer, or with more than one window size, has no plan and runs layer by layer as before;
so does every step that is not "one token a sequence, at most 64 sequences".
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_longlong, c_void_p

import numpy as np
import torch

from . import build
from .ops import KernelError, _check, _ptr, _stream, sm_count

SOURCE = "decode_stack.cu"
HEAD_DIMS = (64, 128)
W_ROWS = 256                  # weight rows of a unit of a product (the kernel's W_ROWS)
# Off unless asked for: measured at Qwen3-8B layer sizes it is slower than the layer-by-layer path at every
# batch and context tried (12 layers, 2,084 positions: 1.73 against 1.24 ms a step at batch 8; 1.76 against
# 1.11 at batch 1; 3.04 against 2.28 at batch 64), because its nine grid barriers a layer and the short
# phases between them cost more than the launches they replace.
ENABLED = os.environ.get("ULTIMA_DECODE_STACK", "0") != "0"
TRACE = os.environ.get("ULTIMA_STACK_TRACE", "0") != "0"        # times of the phases of CTA 0, for measurements
_libs: dict = {}

PH_NORM, PH_GEMM, PH_ATTN, PH_MERGE, PH_SILU = range(5)

# the kernel's Phase record (csrc/decode_stack.cu), field for field
PHASE = np.dtype([
    ("type", "<i4"), ("pad0", "<i4"),
    ("map_w", "<i4"), ("map_b", "<i4"), ("N", "<i4"), ("K", "<i4"), ("out", "<u8"), ("ldo", "<i8"),
    ("w", "<u8"), ("h", "<u8"), ("width", "<i4"), ("eps", "<f4"), ("zero", "<u8"), ("zero_n", "<i8"),
    ("gu", "<u8"), ("act", "<u8"), ("F", "<i4"), ("pad1", "<i4"),
    ("qkv", "<u8"), ("qw", "<u8"), ("kw", "<u8"), ("cs", "<u8"), ("sn", "<u8"), ("kcache", "<u8"), ("vcache", "<u8"),
    ("part_o", "<u8"), ("part_ml", "<u8"), ("o", "<u8"),
    ("nh", "<i4"), ("nkv", "<i4"), ("window", "<i4"), ("ring", "<i4"), ("pages_per_seq", "<i4"), ("map_k", "<i4"),
    ("map_v", "<i4"), ("table", "<i4"), ("c", "<f4"), ("pad2", "<i4")], align=True)


def target(head_dim: int):
    return (SOURCE, (f"HEAD_DIM={int(head_dim)}",))


def lib(head_dim: int):
    L = _libs.get(head_dim)
    if L is None:
        L = build.load(*target(head_dim))
        L.ub_stack_map_2d.argtypes = [c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_int]
        L.ub_stack_map_2d.restype = c_int
        L.ub_decode_stack.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        L.ub_decode_stack.restype = c_int
        L.ub_stack_max_maps.restype = c_int
        L.ub_stack_phase_bytes.restype = c_int
        L.ub_stack_head_dim.restype = c_int
        if L.ub_stack_head_dim() != head_dim or L.ub_stack_phase_bytes() != PHASE.itemsize:
            raise KernelError("the layer-stack library does not match its Python description "
                              f"(head size {L.ub_stack_head_dim()}, phase record of {L.ub_stack_phase_bytes()} bytes)")
        _libs[head_dim] = L
    return L


def token_tile(T: int) -> int:
    return 16 if T <= 16 else 32 if T <= 32 else 64


class _Maps:
    """Tensor maps of a program, made on the host and kept in one device array."""

    def __init__(self, L):
        self.L, self.raw, self.keep = L, [], {}

    def add(self, t: torch.Tensor, box_rows: int) -> int:
        key = (t.data_ptr(), tuple(t.shape), t.stride(0), box_rows)
        if key in self.keep:
            return self.keep[key]
        assert t.dim() == 2 and t.dtype == torch.bfloat16 and t.stride(1) == 1
        buf = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(buf) + 63) & ~63
        rc = self.L.ub_stack_map_2d(addr, t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
        if rc != 0:
            raise KernelError(f"tensor map for a {list(t.shape)} matrix could not be made (code {rc})")
        self.raw.append(ctypes.string_at(addr, 128))
        self.keep[key] = len(self.raw) - 1
        return self.keep[key]

    def on_host(self):
        """(buffer that keeps them alive, address of the first map, count): 64-byte aligned, side by side."""
        buf = ctypes.create_string_buffer(128 * len(self.raw) + 64)
        addr = (ctypes.addressof(buf) + 63) & ~63
        ctypes.memmove(addr, b"".join(self.raw), 128 * len(self.raw))
        return buf, addr, len(self.raw)


class StackPlan:
    """What the layer-stack kernel needs of one model: checked once, programs made for each token tile."""

    def __init__(self, model, rt, cache):
        self.model, self.rt, self.cache = model, rt, cache
        self.head_dim = model.layers[0].mixer.hd
        self.L = lib(self.head_dim)
        self.n_ctas = sm_count(rt.device)
        self.programs: dict = {}
        windows = sorted({int(L.mixer.window) for L in model.layers if L.mixer.window})
        self.window_b = windows[0] if windows else 0

    # ---- may this model run as one kernel? ----------------------------------------------
    @staticmethod
    def fits(model, rt, cache) -> bool:
        from ..parts.arrangement import PreNorm
        from ..parts.attention import Attention
        from ..parts.mlp import GatedSiLU
        from ..parts.norm import RMSNorm
        if not ENABLED or rt.dtype != torch.bfloat16 or not rt.use_tensor_cores or not model.layers:
            return False
        hd = None
        windows = set()
        for L in model.layers:
            if type(L.arrangement) is not PreNorm:
                return False
            if type(L.mixer_norm) is not RMSNorm or type(L.feed_forward_norm) is not RMSNorm:
                return False
            a, f = L.mixer, L.feed_forward
            if type(a) is not Attention or type(f) is not GatedSiLU:
                return False
            if a.hd not in HEAD_DIMS or (hd is not None and a.hd != hd) or a.nh // a.nkv > 16:
                return False
            hd = a.hd
            if a.wqkv.dtype != torch.bfloat16 or a.wo.dtype != torch.bfloat16 or a.width % 8 or a.q_width % 8:
                return False
            if a.position is not None:
                rot = a.position.rotation()
                if rot is None or rot.dim != a.hd or rot.interleaved or not getattr(a.position, "graph_safe", False):
                    return False
            if not getattr(f, "interleaved", False) or f.wgu.dtype != torch.bfloat16 or f.wd.dtype != torch.bfloat16:
                return False
            if a.window:
                windows.add(int(a.window))
        if len(windows) > 1 or len(cache.kv_groups) > 4:
            return False
        # tensor maps travel in the launch's parameters: four weights and the run's two cache maps a run, and
        # three maps of the step's own buffers
        if 6 * len(model.spec.runs) + 3 > lib(hd).ub_stack_max_maps():
            return False
        return all(g.k.dtype == torch.bfloat16 for g in cache.kv_groups)

    # ---- the program of one token tile ----------------------------------------------------
    def _program(self, bn: int):
        prog = self.programs.get(bn)
        if prog is not None:
            return prog
        model, rt, dev, hd = self.model, self.rt, self.rt.device, self.head_dim
        maps = _Maps(self.L)
        width = model.spec.width
        q_max = max(L.mixer.q_width for L in model.layers)
        qkv_max = max(L.mixer.q_width + 2 * L.mixer.kv_width for L in model.layers)
        f_max = max(L.feed_forward.inner for L in model.layers)
        nkv_max = max(L.mixer.nkv for L in model.layers)
        keep = {
            "h": torch.zeros((bn, width), dtype=torch.bfloat16, device=dev),
            "o": torch.zeros((bn, q_max), dtype=torch.bfloat16, device=dev),
            "act": torch.zeros((bn, f_max), dtype=torch.bfloat16, device=dev),
            "qkv": torch.zeros((bn, qkv_max), dtype=torch.float32, device=dev),
            "gu": torch.zeros((bn, 2 * f_max), dtype=torch.float32, device=dev),
            "part_o": torch.zeros((bn * nkv_max + self.n_ctas + 1, 16, hd), dtype=torch.float32, device=dev),
            "part_ml": torch.zeros((bn * nkv_max + self.n_ctas + 1, 16, 2), dtype=torch.float32, device=dev),
            "counter": torch.zeros(1, dtype=torch.int32, device=dev),
        }
        rows = []

        def phase(**kw):
            r = np.zeros((), dtype=PHASE)
            for k, v in kw.items():
                r[k] = v
            rows.append(r)

        for i, run in enumerate(model.spec.runs):
            L = model.layers[run.layer]
            a, f = L.mixer, L.feed_forward
            rc = self.cache.run_cache(i, [None] * len(self.cache.kv_groups))
            kv = rc.kv
            group = self.cache.kv_groups.index(self.cache._kv_of_run[i if rc.owner else run.cache_from])
            n_qkv = a.q_width + 2 * a.kv_width
            h_in = keep["h"][:, :a.width]
            qkv = keep["qkv"][:, :n_qkv]
            # the buffers are wider than this layer may need: views with the layer's own row length
            qkv_flat = keep["qkv"].view(-1)[:bn * n_qkv].view(bn, n_qkv)
            o_flat = keep["o"].view(-1)[:bn * a.q_width].view(bn, a.q_width)
            act_flat = keep["act"].view(-1)[:bn * f.inner].view(bn, f.inner)
            gu_flat = keep["gu"].view(-1)[:bn * 2 * f.inner].view(bn, 2 * f.inner)
            del h_in, qkv
            rot = a.position.rotation() if a.position is not None else None
            att = dict(qkv=qkv_flat.data_ptr(), qw=_ptr(a.q_norm), kw=_ptr(a.k_norm),
                       cs=_ptr(rot.cos) if rot is not None else 0, sn=_ptr(rot.sin) if rot is not None else 0,
                       kcache=kv.k.data_ptr() if kv.owner else 0, vcache=kv.v.data_ptr() if kv.owner else 0,
                       part_o=keep["part_o"].data_ptr(), part_ml=keep["part_ml"].data_ptr(), o=o_flat.data_ptr(),
                       nh=a.nh, nkv=a.nkv, window=int(a.window or 0), ring=kv.ring, pages_per_seq=kv.ring // 64,
                       map_k=maps.add(kv.k.view(-1, hd), 64), map_v=maps.add(kv.v.view(-1, hd), 64), table=group,
                       c=float(a.scale) * 1.4426950408889634, eps=a.eps)
            phase(type=PH_NORM, w=L.mixer_norm.weight.data_ptr(), h=keep["h"].data_ptr(), width=a.width,
                  eps=L.mixer_norm.eps, zero=qkv_flat.data_ptr(), zero_n=bn * n_qkv)
            phase(type=PH_GEMM, map_w=maps.add(a.wqkv, W_ROWS), map_b=maps.add(keep["h"], bn), N=n_qkv, K=a.width,
                  out=qkv_flat.data_ptr(), ldo=n_qkv)
            phase(type=PH_ATTN, **att)
            phase(type=PH_MERGE, **att)
            phase(type=PH_GEMM, map_w=maps.add(a.wo, W_ROWS), map_b=maps.add(o_flat, bn), N=a.width, K=a.q_width, out=0, ldo=a.width)
            phase(type=PH_NORM, w=L.feed_forward_norm.weight.data_ptr(), h=keep["h"].data_ptr(), width=f.width,
                  eps=L.feed_forward_norm.eps, zero=gu_flat.data_ptr(), zero_n=bn * 2 * f.inner)
            phase(type=PH_GEMM, map_w=maps.add(f.wgu, W_ROWS), map_b=maps.add(keep["h"], bn), N=2 * f.inner, K=f.width,
                  out=gu_flat.data_ptr(), ldo=2 * f.inner)
            phase(type=PH_SILU, gu=gu_flat.data_ptr(), act=act_flat.data_ptr(), F=f.inner)
            phase(type=PH_GEMM, map_w=maps.add(f.wd, W_ROWS), map_b=maps.add(act_flat, bn), N=f.width, K=f.inner, out=0, ldo=f.width)
        phases = torch.from_numpy(np.stack(rows).view(np.uint8).reshape(-1).copy()).to(dev)
        prog = {"phases": phases, "n": len(rows), "maps": maps.on_host(), "keep": keep,
                "types": [int(r["type"]) for r in rows],
                "trace": torch.zeros(len(rows) + 1, dtype=torch.int64, device=dev) if TRACE else None}
        self.programs[bn] = prog
        return prog

    # ---- a step ------------------------------------------------------------------------------
    def run(self, x: torch.Tensor, batch) -> None:
        """Run every layer on the residual stream x (float32 [T, width]) in place, for a step of one token a
        sequence; the cache is extended as the layer-by-layer path would extend it."""
        T = batch.n_tokens
        bn = token_tile(T)
        prog = self._program(bn)
        prog["keep"]["counter"].zero_()
        tables = [_ptr(t) for t in batch.tables] + [0] * (4 - len(batch.tables))
        self.rt.launches += 1
        rc = self.L.ub_decode_stack(_ptr(prog["phases"]), prog["n"], prog["maps"][1], prog["maps"][2], T, bn, _ptr(x), _ptr(batch.seq_before),
                                    tables[0], tables[1], tables[2], tables[3], self.window_b,
                                    _ptr(prog["keep"]["counter"]), _ptr(self.rt.status[1:2]), self.n_ctas,
                                    _ptr(prog["trace"]), _stream())
        _check(rc, "decode_stack")

    def phase_times(self, bn: int):
        """(type, microseconds) of every phase of the last launch with token tile ``bn``, as CTA 0 saw them
        (needs ULTIMA_STACK_TRACE=1)."""
        prog = self.programs[bn]
        t = prog["trace"].cpu().numpy()
        return [(prog["types"][i], (t[i + 1] - t[i]) / 1e3) for i in range(prog["n"])]
