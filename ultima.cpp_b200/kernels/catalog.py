"""Which libraries exist: every (source, defines) pair the package may load."""
from __future__ import annotations

PLAIN = [("basic.cu", ()), ("gemm_simt.cu", ()), ("attn_simple.cu", ()), ("sampling.cu", ()),
         ("gemm_tcgen05.cu", ())]
# the tensor-core attention library is built for each head size; these are the sizes that the
# tests, the bench and the usual checkpoints use (any other multiple of 16 is built on demand)
HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128, 256)


TC_HEAD_DIMS = (64, 128)          # head sizes the tcgen05 prefill attention is written for


def all_targets() -> list:
    return (list(PLAIN) + [("attn_mma.cu", (f"HEAD_DIM={hd}",)) for hd in HEAD_DIMS]
            + [("attn_tcgen05.cu", (f"HEAD_DIM={hd}",)) for hd in TC_HEAD_DIMS]
            + [("decode_stack.cu", (f"HEAD_DIM={hd}",)) for hd in TC_HEAD_DIMS])


def targets_for_model(spec, dtype, sampler: bool = True) -> list:
    """What one model needs: the row-wise kernels and the CUDA-core product always (the latter stands
    in for shapes the tensor-core product refuses), the tcgen05 product on the bfloat16 path, and
    whatever the model's parts ask for themselves (``Part.kernel_needs``: the attention part names
    the attention library of its head size).  ``sampler``: the sampling kernel too (a replay of
    given tokens samples nothing)."""
    import torch
    out = [("basic.cu", ()), ("gemm_simt.cu", ())]
    if dtype == torch.bfloat16:
        out.append(("gemm_tcgen05.cu", ()))
    for t in spec.kernel_needs(dtype):
        if t not in out:
            out.append(t)
    if sampler:
        out.append(("sampling.cu", ()))
    return out
