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
            + [("attn_tcgen05.cu", (f"HEAD_DIM={hd}",)) for hd in TC_HEAD_DIMS])


def targets_for_model(spec, dtype, sampler: bool = True) -> list:
    """What one model needs: on the float32 path the CUDA-core product and the float32 attention; on
    the bfloat16 path the tcgen05 product (the CUDA-core one stands in for shapes it refuses) and the
    attention library of each head size the model's mixers use.  ``sampler``: the sampling kernel
    too (a replay of given tokens samples nothing)."""
    import torch
    out = [("basic.cu", ()), ("gemm_simt.cu", ())]
    dims = sorted({L.mixer.get("head_dim") for L in spec.layers if L.mixer.get("head_dim")})
    if dtype == torch.bfloat16:
        out.append(("gemm_tcgen05.cu", ()))
        fits = [hd for hd in dims if hd % 16 == 0 and 16 <= hd <= 256]
        out += [("attn_mma.cu", (f"HEAD_DIM={hd}",)) for hd in fits]
        out += [("attn_tcgen05.cu", (f"HEAD_DIM={hd}",)) for hd in fits if hd in TC_HEAD_DIMS]
        if len(fits) != len(dims):
            out.append(("attn_simple.cu", ()))
    else:
        out.append(("attn_simple.cu", ()))
    if sampler:
        out.append(("sampling.cu", ()))
    return out
