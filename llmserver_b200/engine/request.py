"""A request and its lifecycle: WAITING -> PREFILL -> DECODING -> FINISHED | CANCELLED.

Same state machine as the reference (utils/request.py:5-121), for a token-id engine: no text, no
output queue.  Preemption puts a request back to WAITING with nothing computed; if it had been
decoding it then prefills ``prompt + generated[:-1]`` and does not sample again at the end, so no
token is produced twice (utils/request.py:63-75).
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
    pass


class Request:
    def __init__(self, request_id: str, prompt_token_ids: List[int], max_new_tokens: int, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False):
        if not prompt_token_ids:
            raise ValueError("prompt_token_ids must not be empty")
        if max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens is <= 0: {max_new_tokens}")
        if temperature < 0:
            raise ValueError(f"temperature must not be negative: {temperature}")
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.generated_token_ids: List[int] = []
        self.max_new_tokens = max_new_tokens
        self.temperature = float(temperature)
        self.seed = int(seed)
        self.ignore_eos = ignore_eos
        self.num_computed_tokens = 0
        self.prefix_idle_pages = 0     # idle cached pages a shared prefix would take back into use
        self.status = RequestStatus.WAITING
        self.finish_reason: Optional[RequestFinishReason] = None
        self.created_at = time.time()
        self.first_token_at: Optional[float] = None
        self.finished_at: Optional[float] = None
        self.needs_decode_resume = False
        self.waiting_steps = 0
        self.preemption_count = 0

    @property
    def prefill_token_ids(self) -> List[int]:
        if self.needs_decode_resume:
            return self.prompt_token_ids + self.generated_token_ids[:-1]
        return self.prompt_token_ids

    @property
    def remaining_prefill(self) -> int:
        return len(self.prefill_token_ids) - self.num_computed_tokens

    def preempt_for_compute(self) -> None:
        if self.status not in (RequestStatus.PREFILL, RequestStatus.DECODING):
            raise RequestStateError(f"Request cannot be preempted, current request status is {self.status.value}")
        self.needs_decode_resume = self.needs_decode_resume or self.status == RequestStatus.DECODING
        self.status = RequestStatus.WAITING
        self.num_computed_tokens = 0
        self.prefix_idle_pages = 0
        self.preemption_count += 1

    def start_prefill(self) -> None:
        if self.status != RequestStatus.WAITING:
            raise RequestStateError(f"Request cannot be put for prefill, current request status is {self.status.value}")
        self.status = RequestStatus.PREFILL

    def advance_prefill(self, num_tokens: int) -> None:
        if self.status != RequestStatus.PREFILL:
            raise RequestStateError(f"Request prefill cannot advance, current request status is {self.status.value}")
        if num_tokens <= 0 or num_tokens > self.remaining_prefill:
            raise ValueError(f"Invalid number of prefill tokens: num_tokens: {num_tokens}, remaining_prompt: {self.remaining_prefill}")
        self.num_computed_tokens += num_tokens

    def complete_prefill(self) -> None:
        if self.status != RequestStatus.PREFILL:
            raise RequestStateError(f"Request prefill cannot be completed, current request status is {self.status.value}")
        if self.remaining_prefill != 0:
            raise RequestStateError("Request prefill cannot be completed before all prompt tokens are computed: "
                                    f"num_computed_tokens: {self.num_computed_tokens}, prompt_tokens: {len(self.prefill_token_ids)}")
        self.status = RequestStatus.DECODING
        self.needs_decode_resume = False

    def append_generated_token(self, token_id: int) -> None:
        if self.status != RequestStatus.DECODING:
            raise RequestStateError(f"Request is not in the decoding stage: current request status is {self.status.value}")
        if self.first_token_at is None:
            self.first_token_at = time.time()
        self.generated_token_ids.append(int(token_id))

    def complete_decode(self) -> None:
        if self.status != RequestStatus.DECODING:
            raise RequestStateError(f"Request decoding cannot be completed, it is not in the decoding stage: current request status is {self.status.value}")
        self.num_computed_tokens += 1

    def finish(self, finish_reason) -> None:
        if self.status in (RequestStatus.FINISHED, RequestStatus.CANCELLED):
            raise RequestStateError(f"Request cannot be finished, it has already been finished or cancelled: current request status is {self.status.value}")
        self.status = RequestStatus.FINISHED
        self.finish_reason = RequestFinishReason(finish_reason)
        self.finished_at = time.time()

    def cancel(self) -> None:
        self.status = RequestStatus.CANCELLED
        self.finish_reason = RequestFinishReason.CANCELLED
        self.finished_at = time.time()
