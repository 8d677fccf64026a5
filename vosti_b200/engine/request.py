"""Requests as the scheduler keeps them.

Fields and the finish rule follow the reference's request state
(src/exec/request_state.rs:192-226, 476-501): a request carries its id, prompt tokens,
generation budget, up to three end-of-sequence ids and an ignore-EOS flag; it is
finished when it has generated `max_tokens` tokens or (unless EOS is ignored) the token
just emitted is one of its EOS ids. Temperature and seed are added here; the reference's
sampler state is empty because it only samples greedily (src/boundary/sampler.rs:7-19).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

MAX_EOS_TOKEN_IDS = 3


class AdmissionStatus(enum.Enum):
    """Why a request was or was not taken (src/exec/request_state.rs:203-211)."""

    ACCEPTED = "accepted"
    DUPLICATE_ID = "duplicate request id"
    EMPTY_PROMPT = "empty prompt"
    BAD_EOS = "the EOS id list must hold one to three ids"
    ZERO_BUDGET = "max_tokens must be positive"
    TOO_LONG = "prompt plus max_tokens exceeds the context limit"
    BAD_TOKEN = "a prompt token is outside the vocabulary"
    BAD_SAMPLING = "temperature must be finite and >= 0"


@dataclass
class Request:
    request_id: object
    prompt_tokens: List[int]
    max_tokens: int
    eos_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False
    temperature: float = 0.0
    seed: int = 0
    generated: List[int] = field(default_factory=list)
    computed: int = 0              # tokens whose cache entries exist
    preemptions: int = 0
    finished: bool = False
    finish_reason: str = ""

    def tokens(self) -> List[int]:
        return self.prompt_tokens + self.generated

    def token_range(self, start: int, count: int) -> List[int]:
        """tokens()[start:start + count] without building the whole list."""
        p = len(self.prompt_tokens)
        if start >= p:
            return self.generated[start - p:start - p + count]
        if start + count <= p:
            return self.prompt_tokens[start:start + count]
        return self.prompt_tokens[start:] + self.generated[:start + count - p]

    def num_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.generated)

    def remaining(self) -> int:
        """Known tokens whose cache entries do not exist yet (1 while decoding)."""
        return self.num_tokens() - self.computed

    def is_decoding(self) -> bool:
        return bool(self.generated) and self.remaining() == 1

    def record(self, token: int) -> bool:
        """Append a sampled token; returns whether the request is now finished."""
        self.generated.append(int(token))
        if len(self.generated) >= self.max_tokens:
            self.finished, self.finish_reason = True, "length"
        elif not self.ignore_eos and int(token) in self.eos_token_ids:
            self.finished, self.finish_reason = True, "eos"
        return self.finished
