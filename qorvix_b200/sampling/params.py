"""Sampling parameters with the reference's names, defaults and disabled values
(runtime/include/qorvix/runtime/sampler.hpp:12-21): temperature <= 0 is greedy; top_k == 0,
top_p >= 1 and min_p <= 0 switch that filter off; penalties of 1 / 0 / 0 do nothing."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repetition_penalty: float = 1.1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    penalty_last_n: int = 64
    seed: int = 0
    max_new_tokens: int = 128          # the reference's GenerationConfig::maxNewTokens (generator.hpp:19)
    ignore_eos: bool = False
    stop_token_ids: Tuple[int, ...] = ()

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return self.penalty_last_n != 0 and (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                                             or self.presence_penalty != 0.0)

    @staticmethod
    def greedy_params(max_new_tokens: int = 128, **kw) -> "SamplingParams":
        return SamplingParams(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                              max_new_tokens=max_new_tokens, **kw)
