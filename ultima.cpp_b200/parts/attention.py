"""The attention mixer: grouped-query attention over the cache, with optional per-head norm
of queries and keys, an optional position encoding (any part of the "position" family) and an
optional window."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Mixer, KVNeed, PartSpec, build_part, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    """q, k, v projections (no bias), per-head RMSNorm of q and k before the rotation when
    ``qk_norm`` (one weight of head size for all heads, the layer's eps), rotation, write of
    k and v into the cache before reading so a token sees itself, softmax(q k / sqrt(d)) v
    with query head h on KV head h // (heads / kv heads), output projection added to the
    residual stream.  Reference: src/model/qwen_block.cpp:682-690, :713-727, :732-751,
    :775-783, :94-135.

    The three projections are held as one matrix [q | k | v] and run as one product.
    """

    @property
    def graph_safe(self) -> bool:
        """Launches kernels only, no host work that depends on the data; a position encoding it holds
        has to say the same of itself."""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, qk_norm: bool,
                 eps: float, position: PartSpec | None, window: int | None = None,
                 scale: float | None = None):
        if n_heads % n_kv_heads:
            raise ValueError("heads must be a multiple of kv heads")
        self.width, self.nh, self.nkv, self.hd = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        self.qk_norm, self.eps, self.window = bool(qk_norm), float(eps), window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        self.position = build_part("position", position) if position is not None else None
        self.q_width, self.kv_width = self.nh * self.hd, self.nkv * self.hd
        self.wqkv = self.wo = self.q_norm = self.k_norm = None

    def weight_specs(self):
        s = [WeightSpec("q_proj.weight", (self.q_width, self.width)),
             WeightSpec("k_proj.weight", (self.kv_width, self.width)),
             WeightSpec("v_proj.weight", (self.kv_width, self.width)),
             WeightSpec("o_proj.weight", (self.width, self.q_width))]
        if self.qk_norm:
            s += [WeightSpec("q_norm.weight", (self.hd,), "vector", ("one_plus_normal", 0.05)),
                  WeightSpec("k_norm.weight", (self.hd,), "vector", ("one_plus_normal", 0.05))]
        return s

    def cache_need(self):
        return KVNeed(self.nkv, self.hd, self.window)

    def kernel_needs(self, run_dtype):
        from ..kernels import attn_tc, catalog
        if run_dtype != torch.bfloat16:
            return [("attn_simple.cu", ())]
        if self.hd % 16 == 0 and 16 <= self.hd <= 256:
            out = [attn_tc.target(self.hd)]
            if self.hd in catalog.TC_HEAD_DIMS:
                out.append(attn_tc.tc_target(self.hd))
            return out
        return [("attn_simple.cu", ())]

    def bind(self, tensors, rt):
        if self.hd % 2 or self.hd > ops.MAX_HEAD_DIM:
            raise ValueError(f"attention: head size {self.hd} is not one the kernels take (even, at most "
                             f"{ops.MAX_HEAD_DIM})")
        ws = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v projections must share one element type")
        self.wqkv = torch.cat(ws, dim=0).contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        if self.qk_norm:
            self.q_norm = tensors["q_norm.weight"].float().contiguous()
            self.k_norm = tensors["k_norm.weight"].float().contiguous()
        if self.position is not None:
            self.position.bind({}, rt)

    def forward(self, h, residual, batch, cache, rt):
        T = h.shape[0]
        kv = cache.kv
        # A position encoding that describes itself as a rotation of pairs is applied by the kernels
        # that norm and write the cache; any other is called between the norm and the cache write.
        rot = self.position.rotation() if self.position is not None else None
        apart = self.position is not None and rot is None
        cos, sin = (rot.cos, rot.sin) if rot is not None else (None, None)
        whole = rot is None or (rot.dim == self.hd and not rot.interleaved)
        o = rt.arena.alloc((T, self.q_width), rt.dtype)
        parts = rt.matmul_parts(h, self.wqkv)        # few tokens: K in slices, summed by the next kernel
        if parts is not None:
            # one token a sequence: the attention kernel can take the slices as they are
            if not apart and whole and rt.attention_from_qkv(parts, self.q_norm, self.k_norm, cos, sin, self.eps, kv,
                                                             o, batch, self.nh, self.nkv, self.hd, self.scale):
                rt.matmul(o, self.wo, residual, ops.EPI_ADD)
                return
            qkv = parts
            q = rt.arena.alloc((T, self.q_width), rt.dtype)
        else:
            qkv = rt.arena.alloc((T, self.q_width + 2 * self.kv_width), rt.dtype)
            rt.matmul(h, self.wqkv, qkv)
            q = qkv[:, :self.q_width]
        rt.launches += 1
        if apart:
            kbuf = rt.arena.alloc((2, T, self.kv_width), q.dtype)
            ops.qk_prepare(qkv, self.q_norm, self.k_norm, None, None, batch.tok_pos, batch.tok_seq,
                           kv.k, kv.v, kv.table, kv.ring, kv.page, self.nh, self.nkv, self.hd, self.eps,
                           write_kv=kv.owner, q_out=q, kv_out=(kbuf[0], kbuf[1]))
            self.position.forward(q.view(T, self.nh, self.hd), kbuf[0].view(T, self.nkv, self.hd), batch.tok_pos, rt)
            if kv.owner:
                rt.launches += 1
                ops.kv_write(kbuf[0], kbuf[1], batch.tok_pos, batch.tok_seq, kv.k, kv.v, kv.table, kv.ring, kv.page,
                             self.nkv, self.hd)
        else:
            ops.qk_prepare(qkv, self.q_norm, self.k_norm, cos, sin, batch.tok_pos, batch.tok_seq,
                           kv.k, kv.v, kv.table, kv.ring, kv.page, self.nh, self.nkv, self.hd, self.eps,
                           write_kv=kv.owner, q_out=q, rotary_dim=rot.dim if rot is not None else None,
                           interleaved=bool(rot.interleaved) if rot is not None else False)
        rt.attention(q, kv, o, batch, self.nh, self.nkv, self.hd, self.scale)
        rt.matmul(o, self.wo, residual, ops.EPI_ADD)
