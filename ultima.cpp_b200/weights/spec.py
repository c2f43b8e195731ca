"""What a part asks of the weight file: names, shapes and how a random one is drawn."""
from __future__ import annotations

from dataclasses import dataclass


class WeightError(ValueError):
    """Missing, unexpected or mis-shaped tensors; one error lists all of them."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


@dataclass(frozen=True)
class WeightSpec:
    """One tensor of the file.

    kind:  "matrix" (a projection or the embedding table: kept in the file's 16-bit
           type on the bfloat16 path), "vector" (a norm's weight: small, held in 32-bit),
           "table" (an integer table: held as int32).
    init:  ("normal", std) or ("one_plus_normal", std) or ("zeros",) for the random mode.
    """
    name: str
    shape: tuple
    kind: str = "matrix"
    init: tuple = ("normal", 0.02)
