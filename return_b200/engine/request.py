"""A generation request and its result, with the reference's field names.

``Request`` mirrors rollout/engine.py:13-63: ``id``, ``prompt_ids``, ``max_new_tokens`` (32),
``temperature`` (1.0; <= 0 is greedy), ``top_p`` (1.0), ``top_k`` (0 = off), ``stop_ids`` (a list of
token *sequences*; generation ends when the output ends with one of them, and the stop tokens
stay in the output, :49-57), ``output``, ``output_logprobs``.  The paragraph fields of the reference
(``split_ids``, ``subs``, ``swap``, ...) belong to its context-folding feature and have no counterpart.
``seed`` is new: the random draws of a request come from (seed, index of the output token) alone.
``keep``: what the request holds in the cache stays when it ends, for a later request with the same id
whose prompt begins with this one's prompt and output (the reference keeps every session until
``release``, rollout/engine.py:266-306; here None takes the engine's setting).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional


@dataclass
class Request:
    id: Hashable
    prompt_ids: List[int]
    max_new_tokens: int = 32
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    stop_ids: List[List[int]] = field(default_factory=list)
    seed: Optional[int] = None
    keep: Optional[bool] = None
    output: List[int] = field(default_factory=list)
    output_logprobs: List[float] = field(default_factory=list)
    finish_reason: Optional[str] = None          # "length" | "stop" | "error"
    error: Optional[BaseException] = None
    # scheduler state
    num_computed: int = 0                        # tokens of prompt + output whose keys are cached
    num_preemptions: int = 0
    arrival: int = 0

    def push(self, tok: int, logprob: float = 0.0) -> None:
        self.output.append(int(tok))
        self.output_logprobs.append(float(logprob))

    @property
    def last_token(self) -> int:
        return self.output[-1]

    @property
    def all_ids(self) -> List[int]:
        return list(self.prompt_ids) + self.output

    def ids_slice(self, start: int, stop: int) -> List[int]:
        """Tokens [start, stop) of prompt + output without building the whole list."""
        n = len(self.prompt_ids)
        if start >= n:
            return self.output[start - n:stop - n]
        if stop <= n:
            return list(self.prompt_ids[start:stop])
        return list(self.prompt_ids[start:]) + self.output[:stop - n]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output)

    @property
    def finished(self) -> bool:
        """Length reached, or the output ends with a stop sequence (rollout/engine.py:49-57)."""
        if len(self.output) >= self.max_new_tokens:
            return True
        for seq in self.stop_ids:
            n = len(seq)
            if n and len(self.output) >= n and self.output[-n:] == list(seq):
                return True
        return False

    def reason(self) -> str:
        """"length" if the budget of new tokens is used up, else "stop" (rollout/engine_actor.py:70-71)."""
        return "length" if len(self.output) >= self.max_new_tokens else "stop"


@dataclass
class GenerationResult:
    """What a finished request gives back (the reference's result dict, rollout/engine_actor.py:73-78)."""
    id: Hashable
    output_ids: List[int]
    output_logprobs: List[float]
    num_tokens: int
    finish_reason: str

    def as_dict(self) -> dict:
        return {"output_ids": self.output_ids, "output_logprobs": self.output_logprobs,
                "num_tokens": self.num_tokens, "finish_reason": self.finish_reason}
