"""Which libraries exist: every (source, defines) pair the package may load."""
from __future__ import annotations

PLAIN = [("basic.cu", ()), ("gemm_simt.cu", ()), ("attn_simple.cu", ()), ("sampling.cu", ()),
         ("gemm_tcgen05.cu", ())]


def all_targets() -> list:
    return list(PLAIN)
