"""A generation request and its life: WAITING -> RUNNING -> FINISHED.

Same fields, states and finish rules as the reference's ``Request``
(src/distengine/request.py:4-63): a request ends with reason "eos" when the sampled token equals
``eos_token_id`` and with "length" when ``max_new_tokens`` tokens were generated; an
``eos_token_id`` of -1 never matches (src/utils/capacity.py:22).  Added: temperature and seed for
sampling, and ``num_computed``, the number of its tokens whose keys and values are in the cache.
"""

from __future__ import annotations

from enum import Enum, auto


class RequestStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Request:
    def __init__(self, request_id: str, prompt_token_ids: list[int], max_new_tokens: int,
                 eos_token_id: int, temperature: float = 0.0, seed: int = 0) -> None:
        if not isinstance(request_id, str) or not request_id:
            raise ValueError("request_id must be a nonempty string")
        if type(max_new_tokens) is not int or max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be a positive integer")
        if not isinstance(prompt_token_ids, (list, tuple)) or len(prompt_token_ids) == 0:
            raise ValueError("prompt_token_ids must be a nonempty list")
        if type(eos_token_id) is not int:
            raise ValueError("eos_token_id must be an integer")
        if not isinstance(temperature, (int, float)) or temperature < 0:
            raise ValueError("temperature must be a number >= 0")
        if type(seed) is not int:
            raise ValueError("seed must be an integer")
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.max_new_tokens = max_new_tokens
        self.eos_token_id = eos_token_id
        self.temperature = float(temperature)
        self.seed = seed
        self.generated_token_ids: list[int] = []
        self.reason: str | None = None
        self.status = RequestStatus.WAITING
        self.num_computed = 0
        self.num_preemptions = 0

    @property
    def token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.generated_token_ids

    def tokens_from(self, start: int, count: int) -> list[int]:
        """``token_ids[start: start + count]`` without joining the two lists."""
        p = len(self.prompt_token_ids)
        end = start + count
        if end <= p:
            return self.prompt_token_ids[start:end]
        if start >= p:
            return self.generated_token_ids[start - p: end - p]
        return self.prompt_token_ids[start:] + self.generated_token_ids[: end - p]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.generated_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_generated_tokens(self) -> int:
        return len(self.generated_token_ids)

    @property
    def is_finished(self) -> bool:
        return self.status == RequestStatus.FINISHED

    def append_token(self, token_id: int) -> None:
        if self.status != RequestStatus.RUNNING:
            raise RuntimeError(f"request '{self.request_id}' is {self.status.name}: only a "
                               f"running request takes a new token")
        self.generated_token_ids.append(token_id)
        if token_id == self.eos_token_id:
            self.reason = "eos"
            self.status = RequestStatus.FINISHED
        elif len(self.generated_token_ids) == self.max_new_tokens:
            self.reason = "length"
            self.status = RequestStatus.FINISHED

    def snapshot(self) -> dict:
        """The completion record, as the reference's workers report it
        (src/distengine/worker.py:66-73)."""
        return {"request_id": self.request_id,
                "prompt_token_ids": list(self.prompt_token_ids),
                "generated_token_ids": list(self.generated_token_ids),
                "status": self.status.name, "reason": self.reason}
