"""Sampling parameters with the reference's names, meanings and defaults
(`SampleParams`, src/model/sampler.rs:123-157; CLI defaults src/commands/mod.rs:81-92)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0      # 0 -> greedy argmax (lowest index wins a tie)
    top_p: float = 1.0            # nucleus: smallest set whose mass reaches top_p
    top_k: int = 0                # keep the k largest logits; 0 = off
    min_p: float = 0.0            # drop p < min_p * max p; 0 = off
    frequency_penalty: float = 0.0   # logit -= frequency_penalty * count
    presence_penalty: float = 0.0    # logit -= presence_penalty if the token has appeared
    # token id -> value added to its raw logit before the temperature (-100 bans a token); a mapping
    # or pairs, kept as sorted pairs; ids beyond the vocabulary are passed over (sampler.rs:351-358)
    logit_bias: tuple[tuple[int, float], ...] = ()
    logprobs: bool = False        # return ln p of every chosen token (the distribution before min-p / top-p)
    top_logprobs: int = 0         # and of the n most probable tokens beside it (at most 20; needs logprobs)
    max_tokens: int = 128
    seed: int | None = None       # None: a seed is drawn when the request is added
    eos_token_ids: tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self):
        bias = self.logit_bias
        pairs = bias.items() if hasattr(bias, "items") else bias
        pairs = tuple(sorted((int(t), float(b)) for t, b in pairs))
        if len({t for t, _ in pairs}) != len(pairs) or any(t < 0 for t, _ in pairs):
            raise ValueError("logit_bias: one value per token id, ids >= 0")
        object.__setattr__(self, "logit_bias", pairs)
        if not 0 <= self.top_logprobs <= 20:
            raise ValueError("top_logprobs must be in 0..20")
        if self.top_logprobs and not self.logprobs:
            raise ValueError("top_logprobs needs logprobs=True")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def has_penalties(self) -> bool:
        return self.frequency_penalty != 0.0 or self.presence_penalty != 0.0
