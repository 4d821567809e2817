"""One generation request and where it stands.

The stations are the reference's (utils/request.py:5-121: waiting, prefill, decoding, finished, cancelled) and so
are the public names a caller reads (``request_id``, ``prompt_token_ids``, ``generated_token_ids``, ``status``,
``finish_reason``); it is a token-id request without text or an output queue.  The engine moves a request with four
calls: ``admit`` when it gets a row of the batch, ``ran`` after a step that fed some of its tokens, ``take`` for a
sampled token, ``put_out`` when its pages are needed by older requests.

Being put out loses the cache, not the tokens: the request then has to feed ``prompt + generated[:-1]`` again and
samples nothing at the end of that, because the token that follows is already known, so no token is produced twice
(the rule of utils/request.py:63-75).
"""
from __future__ import annotations

import time
from enum import Enum
from typing import List, Optional


class RequestStatus(Enum):
    WAITING = "Waiting"
    PREFILL = "Prefill"
    DECODING = "Decoding"
    FINISHED = "Finished"
    CANCELLED = "Cancelled"


class RequestFinishReason(Enum):
    EOS = "eos"
    LENGTH = "length"
    CANCELLED = "cancelled"
    ERROR = "error"


class RequestStateError(RuntimeError):
    """A request was asked to do something its station does not allow."""


_LIVE = (RequestStatus.PREFILL, RequestStatus.DECODING)
_OVER = (RequestStatus.FINISHED, RequestStatus.CANCELLED)


class Request:
    def __init__(self, request_id: str, prompt_token_ids: List[int], max_new_tokens: int, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False):
        if len(prompt_token_ids) == 0:
            raise ValueError(f"request {request_id!r} has an empty prompt")
        if max_new_tokens < 1:
            raise ValueError(f"request {request_id!r} asks for {max_new_tokens} new tokens; at least one is needed")
        if temperature < 0:
            raise ValueError(f"request {request_id!r}: a temperature cannot be negative ({temperature})")
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.generated_token_ids: List[int] = []
        self.max_new_tokens = max_new_tokens
        self.temperature, self.seed, self.ignore_eos = float(temperature), int(seed), ignore_eos
        self.status = RequestStatus.WAITING
        self.finish_reason: Optional[RequestFinishReason] = None
        self.num_computed_tokens = 0      # tokens of ``feed`` whose keys and values are in the cache
        self.replaying = False            # put out while decoding: the cache is rebuilt, nothing is sampled at its end
        self.prefix_idle_pages = 0        # idle cached pages a shared prefix would take back into use
        self.times_put_out = 0
        self.steps_queued = 0
        self.created_at = time.time()
        self.first_token_at: Optional[float] = None
        self.finished_at: Optional[float] = None

    # ------------------------------------------------------------------ what has to be fed
    @property
    def feed(self) -> List[int]:
        """The tokens whose keys and values must be cached before the next token can be sampled or decoded."""
        if self.replaying:
            return self.prompt_token_ids + self.generated_token_ids[:-1]
        return self.prompt_token_ids

    @property
    def pending(self) -> int:
        return len(self.feed) - self.num_computed_tokens

    def _require(self, allowed, doing: str) -> None:
        if self.status not in allowed:
            raise RequestStateError(f"request {self.request_id!r} is {self.status.value.lower()}: it cannot {doing}")

    # ------------------------------------------------------------------ moves
    def admit(self) -> None:
        self._require((RequestStatus.WAITING,), "be admitted")
        self.status = RequestStatus.PREFILL

    def ran(self, count: int) -> None:
        """A step ran ``count`` more of this request's tokens.  When the last token of ``feed`` is in, the request
        decodes from then on."""
        self._require(_LIVE, "run tokens")
        if self.status is RequestStatus.DECODING:
            if count != 1:
                raise ValueError(f"request {self.request_id!r} decodes one token a step, not {count}")
            self.num_computed_tokens += 1
            return
        if not 1 <= count <= self.pending:
            raise ValueError(f"request {self.request_id!r}: {count} tokens were run, {self.pending} were pending")
        self.num_computed_tokens += count
        if self.pending == 0:
            self.status = RequestStatus.DECODING
            self.replaying = False

    def take(self, token_id: int) -> None:
        """Appends a sampled token."""
        self._require((RequestStatus.DECODING,), "take a sampled token")
        if self.first_token_at is None:
            self.first_token_at = time.time()
        self.generated_token_ids.append(int(token_id))

    def put_out(self) -> None:
        """Its pages go to others: back to waiting with nothing cached."""
        self._require(_LIVE, "be put out")
        if self.status is RequestStatus.DECODING:
            self.replaying = True
        self.status = RequestStatus.WAITING
        self.num_computed_tokens = 0
        self.prefix_idle_pages = 0
        self.times_put_out += 1

    def finish(self, reason) -> None:
        if self.status in _OVER:
            raise RequestStateError(f"request {self.request_id!r} is over already ({self.status.value.lower()})")
        self.status = RequestStatus.FINISHED
        self.finish_reason = RequestFinishReason(reason)
        self.finished_at = time.time()

    def cancel(self) -> None:
        self.status = RequestStatus.CANCELLED
        self.finish_reason = RequestFinishReason.CANCELLED
        self.finished_at = time.time()
