"""What parts run on: the device, the element type of activations, scratch memory and the
choice of kernel for a matrix product or an attention call.

Parts never pick a kernel by model; they ask the runtime for "a product of these two
matrices with this epilogue" and the runtime picks by element type and shape.
"""
from __future__ import annotations

import torch

from ..kernels import ops


_ELEMENT_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8,
                 torch.uint8: 1, torch.int8: 1, torch.float64: 8, torch.int16: 2, torch.bool: 1}


class Arena:
    """Scratch memory for one step: a bump allocator over one buffer, reset layer by layer.
    A request that does not fit gets a fresh, larger buffer (earlier tensors stay valid
    because they hold their buffer); that happens during warm-up only."""

    ALIGN = 256

    def __init__(self, device, nbytes: int = 1 << 20):
        self.device = device
        self._buf = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        self._off = 0
        self.high_water = 0
        self._retired = []          # earlier buffers stay alive: captured graphs may point into them
        self._views = {}            # (offset, dtype, shape) -> the tensor over that place of the current buffer

    def reserve(self, nbytes: int) -> None:
        if nbytes > self._buf.numel():
            if self._off != 0:
                raise RuntimeError("arena can grow only when empty")
            self._retired.append(self._buf)
            self._views.clear()
            self._buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)

    def mark(self) -> int:
        return self._off

    def reset(self, mark: int = 0) -> None:
        self._off = mark

    def alloc(self, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _ELEMENT_SIZE[dtype]
        start = -(-self._off // self.ALIGN) * self.ALIGN
        if start + nbytes > self._buf.numel():
            size = max(2 * self._buf.numel(), start + nbytes + (1 << 20))
            self._retired.append(self._buf)
            self._views.clear()
            self._buf = torch.empty(size, dtype=torch.uint8, device=self.device)
            start = 0
        self._off = start + nbytes
        if self._off > self.high_water:
            self.high_water = self._off
        # layers reset the arena to the same mark, so the same (place, type, shape) comes again and again:
        # the tensor object made for it the first time is handed out again (making one costs microseconds)
        key = (start, dtype, tuple(shape))
        t = self._views.get(key)
        if t is None:
            if len(self._views) > 4096:
                self._views.clear()
            t = self._views[key] = self._buf[start:start + nbytes].view(dtype).view(*shape)
        return t


class Runtime:
    """dtype: torch.float32 (everything in true 32-bit: CUDA-core products, 32-bit cache) or
    torch.bfloat16 (16-bit activations, weights and cache; 32-bit residual stream, sums,
    softmax, norms and rotation)."""

    def __init__(self, device="cuda:0", dtype=torch.bfloat16, head_dims=()):
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.cache_dtype = dtype
        self.arena = Arena(self.device)
        self._shared: dict = {}
        self.use_tensor_cores = dtype == torch.bfloat16
        self.launches = 0              # kernels of this library launched through the runtime
        # flags the kernels raise: [0] a token id outside the vocabulary, [1] a wait that ran out
        # (they are the head of a buffer whose tail takes the sampled token ids: one copy brings both)
        self.status_and_ids = torch.zeros(4 + 4096, dtype=torch.int32, device=self.device)
        self.status = self.status_and_ids[:4]
        self._status_ptr = self.status[1:2].data_ptr()

    def shared(self, key, make):
        """One object for all parts that ask with the same key (rotation tables and the like)."""
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]

    def check_status(self) -> None:
        """Read the flags the kernels raise (one small copy; waits for the stream)."""
        st = self.status.tolist()
        if any(st):
            self.status.zero_()
            if st[0]:
                raise RuntimeError("a token id outside the vocabulary reached the embedding kernel")
            raise RuntimeError("a wait inside a kernel ran out of time; the step's results are not valid")

    # ---- products ----------------------------------------------------------------------
    def matmul(self, a, w, out, epilogue=ops.EPI_STORE, w2=None):
        """out (=, +=) a @ w.T with float32 accumulation; see kernels.ops for the epilogues."""
        self.launches += 1
        if self.use_tensor_cores and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            from ..kernels import gemm_tc
            key = gemm_tc.launch_key(a, w, out, epilogue, w2, self._status_ptr)
            if gemm_tc.relaunch(key):
                return None
            if gemm_tc.accepts(a, w, out, epilogue, w2):
                return gemm_tc.gemm(a, w, out, epilogue, w2, self, key=key)
        if epilogue == ops.EPI_SWIGLU_IL:
            raise ops.KernelError("the interleaved gate/up layout is for the tensor-core product only; "
                                  "this call does not fit it (operand alignment)")
        return ops.gemm_simt(a, w, out, epilogue, w2)

    def matmul_parts(self, a, w):
        """a @ w.T as a float32 [parts, T, N] whose sum over the first axis is the product (K is cut
        into slices so that a product with few tokens fills the GPU), or None when the product
        is better done whole."""
        if not (self.use_tensor_cores and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            return None
        from ..kernels import gemm_tc
        T, N = a.shape[0], w.shape[0]
        parts = gemm_tc.store_splits(T, N, a.shape[1])
        if parts <= 1:
            return None
        out = self.arena.alloc((parts, T, N), torch.float32)
        if not gemm_tc.accepts(a, w, out[0], ops.EPI_STORE, None):
            return None
        self.launches += 1
        gemm_tc.gemm(a, w, out, ops.EPI_STORE, None, self, splits=parts)
        return out

    # ---- attention ----------------------------------------------------------------------
    def attention_from_qkv(self, qkv_parts, q_norm, k_norm, cos, sin, eps, kv, out, batch, n_heads, n_kv_heads,
                           head_dim, scale) -> bool:
        """Attention of a step of one token a sequence, straight from the float32 partial results of
        the fused q/k/v projection: one kernel sums them, prepares q and the new key, writes the new
        key and value and attends.  False when no kernel takes the case; the caller then prepares
        q and the cache itself and calls ``attention``."""
        if not (self.use_tensor_cores and qkv_parts is not None and batch.max_new == 1):
            return False
        from ..kernels import attn_tc
        done = attn_tc.decode_from_qkv(qkv_parts, q_norm, k_norm, cos, sin, eps, kv, out, batch, n_heads,
                                       n_kv_heads, head_dim, scale, self)
        if done:
            self.launches += 1
        return done

    def attention(self, q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale):
        self.launches += 1
        if self.use_tensor_cores and q.dtype == torch.bfloat16:
            from ..kernels import attn_tc
            if attn_tc.accepts(q, kv, head_dim, n_heads, n_kv_heads):
                return attn_tc.attention(q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, self)
        return ops.attn_simple(q, kv.k, kv.v, out, batch.tok_pos, batch.tok_seq, kv.table, kv.ring,
                               kv.page, n_heads, n_kv_heads, head_dim, kv.window, scale)
