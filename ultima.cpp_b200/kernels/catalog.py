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


def targets_for_model(spec, dtype) -> list:
    """What one model needs: the plain libraries and, on the bfloat16 path, the attention
    library of each head size its mixers use."""
    import torch
    out = list(PLAIN)
    if dtype == torch.bfloat16:
        dims = sorted({L.mixer.get("head_dim") for L in spec.layers if L.mixer.get("head_dim")})
        out += [("attn_mma.cu", (f"HEAD_DIM={hd}",)) for hd in dims if hd % 16 == 0 and hd <= 256]
        out += [("attn_tcgen05.cu", (f"HEAD_DIM={hd}",)) for hd in dims if hd in TC_HEAD_DIMS]
    return out
