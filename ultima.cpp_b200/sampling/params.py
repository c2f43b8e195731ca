"""Sampling parameters, with the reference's names, meanings and defaults.

Fields follow ``SamplerParams`` (include/ultima/sampler/sampler.hpp:16-52) and the JSON keys
of its server (src/server/http_server.cpp:63-81).  ``SamplingParams()`` is the reference's
``identity()`` with temperature 0, which is what its ``run`` command starts from
(apps/ultima-cli/main.cpp:565, :661-664): greedy, every other knob neutral;
``SamplingParams.server_defaults()`` gives the defaults of the struct itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0          # <= 0: first maximum after penalties
    top_k: int = 0                    # 0: off
    top_p: float = 1.0                # >= 1: off
    min_p: float = 0.0                # <= 0: off
    rep_penalty: float = 1.0          # 1: off; divides positive, multiplies negative logits
    repeat_last_n: int = 0            # window of the repetition penalty
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    dry_multiplier: float = 0.0       # 0: off
    dry_base: float = 1.75
    dry_allowed_len: int = 2
    dry_last_n: int = 0
    logit_bias: dict = field(default_factory=dict)     # token id -> added to its logit
    seed: int = 0

    @classmethod
    def server_defaults(cls) -> "SamplingParams":
        return cls(temperature=0.2, top_k=40, top_p=0.95, min_p=0.05, rep_penalty=1.1,
                   repeat_last_n=64, dry_multiplier=0.8, dry_base=1.75, dry_allowed_len=2,
                   dry_last_n=512)

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    @property
    def uses_history(self) -> bool:
        return ((self.rep_penalty != 1.0 and self.repeat_last_n > 0)
                or (self.dry_multiplier > 0.0 and self.dry_last_n > 0)
                or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0)

    def history_window(self) -> int:
        return max(self.repeat_last_n, self.dry_last_n) if self.uses_history else 0

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.rep_penalty <= 0:
            raise ValueError("rep_penalty must be > 0")
        if self.repeat_last_n < 0 or self.dry_last_n < 0 or self.dry_allowed_len < 0:
            raise ValueError("window lengths must be >= 0")
