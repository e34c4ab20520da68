"""CPU request scheduler: waiting -> running -> finished, decode first, strict FIFO admission under
token, request and page budgets, and prompts cut into portions.

The state machine, names and rules are the reference's ``RequestScheduler``
(src/mini_llm_runtime/scheduler.py:96-373): every running request decodes once per step before
anything is admitted (:217-227); waiting prompts are admitted from the head of the queue only, and
the queue stops at the first request that does not fit, never skipping it (:240-262);
``max_mixed_prefill_tokens`` bounds prompt tokens in steps that began with running requests
(:247-255); ``schedule_step`` and ``apply_step_results`` alternate (:207-208); ``abort_step`` puts
newly admitted requests back at the head of the queue and does not consume the step index
(:341-373); EOS wins over the length limit (:318-321).

What is new here is the *portion*: the reference refuses prompts longer than the token budget
(:181-185).  Here a prompt that does not fit the rest of the step's budget is admitted with as
many tokens as fit and stays running, "prefilling", getting further portions in later steps; it
emits its first token in the step that consumes its last prompt token.  ``chunked_prefill=False``
restores the reference's whole-prompt behaviour.

When pages run out the decision is the reference's: the admission callback says no, the request
waits at the head of the queue (and everything behind it waits too) until a finished request
gives pages back; nothing is preempted, swapped or recomputed.  Because admission promises a
request the pages of its whole life, a running request never runs out.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Callable, Collection, Mapping, Sequence
from dataclasses import dataclass, field
from enum import Enum


class RequestStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(str, Enum):
    EOS = "eos"
    MAX_TOKENS = "max_tokens"


class WorkKind(str, Enum):
    PREFILL = "prefill"
    DECODE = "decode"


class BatchingPolicy(str, Enum):
    """CONTINUOUS refills free places while others still run; STATIC waits for the cohort to drain."""

    CONTINUOUS = "continuous"
    STATIC = "static"


@dataclass
class RequestState:
    """What the scheduler knows of one request; it holds no device memory."""

    request_id: str
    prompt_token_ids: tuple[int, ...]
    max_new_tokens: int
    eos_token_ids: frozenset[int]
    arrival_index: int
    temperature: float = 0.0
    seed: int = 0
    status: RequestStatus = RequestStatus.WAITING
    prefill_cursor: int = 0           # prompt tokens already run
    finish_reason: FinishReason | None = None
    _generated_token_ids: list[int] = field(default_factory=list, repr=False)

    @property
    def prefilled(self) -> bool:
        return self.prefill_cursor >= len(self.prompt_token_ids)

    @property
    def generated_token_ids(self) -> tuple[int, ...]:
        return tuple(self._generated_token_ids)

    @property
    def max_cache_tokens(self) -> int:
        # The last generated token is never fed back, so it is never cached
        # (reference: scheduler.py:52-55).
        return len(self.prompt_token_ids) + self.max_new_tokens - 1


@dataclass(frozen=True)
class ScheduledRequest:
    """One request's input to the model in one step."""

    request_id: str
    kind: WorkKind
    input_token_ids: tuple[int, ...]
    emits_token: bool = True          # False for a prompt portion that is not the last
    newly_admitted: bool = False

    @property
    def token_cost(self) -> int:
        return len(self.input_token_ids)


@dataclass(frozen=True)
class SchedulerBatch:
    step_index: int
    items: tuple[ScheduledRequest, ...]
    token_count: int

    @property
    def prefill_request_ids(self) -> tuple[str, ...]:
        return tuple(item.request_id for item in self.items if item.kind is WorkKind.PREFILL)

    @property
    def decode_request_ids(self) -> tuple[str, ...]:
        return tuple(item.request_id for item in self.items if item.kind is WorkKind.DECODE)

    @property
    def admitted_request_ids(self) -> tuple[str, ...]:
        return tuple(item.request_id for item in self.items if item.newly_admitted)

    @property
    def emitting_request_ids(self) -> tuple[str, ...]:
        return tuple(item.request_id for item in self.items if item.emits_token)


@dataclass(frozen=True)
class SchedulerStepUpdate:
    step_index: int
    emitted_tokens: tuple[tuple[str, int], ...]
    finished_request_ids: tuple[str, ...]


class RequestScheduler:
    def __init__(self, *, max_running_requests: int, max_batch_tokens: int,
                 max_mixed_prefill_tokens: int | None = None,
                 admission_callback: Callable[[RequestState], bool] | None = None,
                 batching_policy: BatchingPolicy = BatchingPolicy.CONTINUOUS,
                 chunked_prefill: bool = True) -> None:
        if max_running_requests <= 0 or max_batch_tokens <= 0:
            raise ValueError("max_running_requests and max_batch_tokens must be > 0")
        if max_running_requests > max_batch_tokens:
            raise ValueError("max_running_requests must not exceed max_batch_tokens, or a running "
                             "request could miss its decode step")
        if not isinstance(batching_policy, BatchingPolicy):
            raise ValueError("batching_policy must be a BatchingPolicy")
        if max_mixed_prefill_tokens is not None and (
                isinstance(max_mixed_prefill_tokens, bool) or not isinstance(max_mixed_prefill_tokens, int)
                or max_mixed_prefill_tokens <= 0):
            raise ValueError("max_mixed_prefill_tokens must be a positive integer or None")
        self.max_running_requests = max_running_requests
        self.max_batch_tokens = max_batch_tokens
        self.max_mixed_prefill_tokens = max_mixed_prefill_tokens
        self.batching_policy = batching_policy
        self.chunked_prefill = chunked_prefill
        self._admission_callback = admission_callback
        self._requests: dict[str, RequestState] = {}
        self._waiting: deque[str] = deque()
        self._running: list[str] = []
        self._finished: list[str] = []
        self._next_arrival_index = 0
        self._next_step_index = 0
        self._outstanding: SchedulerBatch | None = None

    # ------------------------------------------------------------------ views
    @property
    def waiting_request_ids(self) -> tuple[str, ...]:
        return tuple(self._waiting)

    @property
    def running_request_ids(self) -> tuple[str, ...]:
        return tuple(self._running)

    @property
    def finished_request_ids(self) -> tuple[str, ...]:
        return tuple(self._finished)

    @property
    def outstanding_batch(self) -> SchedulerBatch | None:
        return self._outstanding

    @property
    def has_unfinished_requests(self) -> bool:
        return bool(self._waiting or self._running or self._outstanding)

    def get_request(self, request_id: str) -> RequestState:
        try:
            return self._requests[request_id]
        except KeyError:
            raise KeyError(f"unknown request_id={request_id!r}") from None

    # ------------------------------------------------------------------ submit
    def submit(self, request_id: str, prompt_token_ids: Sequence[int], *, max_new_tokens: int,
               eos_token_ids: int | Collection[int] | None = None, temperature: float = 0.0,
               seed: int = 0) -> RequestState:
        """Append a request to the waiting queue (allowed while a batch is outstanding)."""
        if not request_id:
            raise ValueError("request_id must not be empty")
        if request_id in self._requests:
            raise ValueError(f"request_id={request_id!r} already exists")
        prompt = self._validate_token_sequence(prompt_token_ids, "prompt_token_ids")
        if not self.chunked_prefill and len(prompt) > self.max_batch_tokens:
            raise ValueError(f"prompt length={len(prompt)} exceeds max_batch_tokens="
                             f"{self.max_batch_tokens} and chunked prefill is off")
        if isinstance(max_new_tokens, bool) or not isinstance(max_new_tokens, int) or max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be a positive integer")
        if not isinstance(temperature, (int, float)) or isinstance(temperature, bool) or temperature < 0:
            raise ValueError("temperature must be a number >= 0 (0 selects greedy)")
        if isinstance(seed, bool) or not isinstance(seed, int) or not 0 <= seed < (1 << 63):
            raise ValueError("seed must be an integer in [0, 2^63)")
        request = RequestState(
            request_id=request_id, prompt_token_ids=prompt, max_new_tokens=int(max_new_tokens),
            eos_token_ids=self._normalize_eos(eos_token_ids), arrival_index=self._next_arrival_index,
            temperature=float(temperature), seed=int(seed))
        self._next_arrival_index += 1
        self._requests[request_id] = request
        self._waiting.append(request_id)
        return request

    # ------------------------------------------------------------------ schedule
    def schedule_step(self) -> SchedulerBatch | None:
        """Decodes of all running requests first, then further portions of running prompts, then
        strict-FIFO admission of waiting prompts with what is left of the budgets."""
        if self._outstanding is not None:
            raise RuntimeError("the previous scheduler batch has not been applied or aborted")
        if not self._running and not self._waiting:
            return None

        items: list[ScheduledRequest] = []
        running_at_step_start = bool(self._running)
        for request_id in self._running:
            request = self._requests[request_id]
            if request.prefilled:
                if not request._generated_token_ids:
                    raise RuntimeError(f"running request {request_id!r} has no prefill result")
                items.append(ScheduledRequest(request_id, WorkKind.DECODE,
                                              (request._generated_token_ids[-1],)))
        token_count = len(items)
        mixed_prefill_tokens = 0

        def portion_budget() -> int:
            budget = self.max_batch_tokens - token_count
            if running_at_step_start and self.max_mixed_prefill_tokens is not None:
                budget = min(budget, self.max_mixed_prefill_tokens - mixed_prefill_tokens)
            return budget

        # Prompts already running go on before anything new is admitted (arrival order).
        for request_id in self._running:
            request = self._requests[request_id]
            if request.prefilled:
                continue
            budget = portion_budget()
            if budget <= 0:
                break
            remaining = len(request.prompt_token_ids) - request.prefill_cursor
            count = min(remaining, budget)
            start = request.prefill_cursor
            items.append(ScheduledRequest(request_id, WorkKind.PREFILL,
                                          request.prompt_token_ids[start:start + count],
                                          emits_token=(count == remaining)))
            token_count += count
            mixed_prefill_tokens += count

        available_slots = self.max_running_requests - len(self._running)
        may_admit = self.batching_policy is BatchingPolicy.CONTINUOUS or not running_at_step_start
        while may_admit and self._waiting and available_slots > 0:
            request_id = self._waiting[0]
            request = self._requests[request_id]
            prompt_cost = len(request.prompt_token_ids)
            budget = portion_budget()
            if self.chunked_prefill:
                if budget <= 0:
                    break
                count = min(prompt_cost, budget)
            else:
                # Whole prompts only: the head of the queue that does not fit stops admission.
                if prompt_cost > budget:
                    break
                count = prompt_cost
            # The callback must have no effect when it answers False and must have reserved the
            # request's resources when it answers True.
            if self._admission_callback is not None and not self._admission_callback(request):
                break
            self._waiting.popleft()
            request.status = RequestStatus.RUNNING
            self._running.append(request_id)
            items.append(ScheduledRequest(request_id, WorkKind.PREFILL, request.prompt_token_ids[:count],
                                          emits_token=(count == prompt_cost), newly_admitted=True))
            token_count += count
            if running_at_step_start:
                mixed_prefill_tokens += count
            available_slots -= 1

        if not items:
            return None
        batch = SchedulerBatch(self._next_step_index, tuple(items), token_count)
        self._next_step_index += 1
        self._outstanding = batch
        return batch

    # ------------------------------------------------------------------ results
    def apply_step_results(self, generated_tokens: Mapping[str, int]) -> SchedulerStepUpdate:
        """Write back one token for every item that emits one; validated before any change."""
        batch = self._outstanding
        if batch is None:
            raise RuntimeError("no scheduler batch is waiting for results")
        expected_ids = batch.emitting_request_ids
        actual_ids = tuple(generated_tokens)
        if set(actual_ids) != set(expected_ids) or len(actual_ids) != len(expected_ids):
            missing = sorted(set(expected_ids) - set(actual_ids))
            extra = sorted(set(actual_ids) - set(expected_ids))
            raise ValueError(f"step results do not match the batch: missing={missing}, extra={extra}")
        validated = {rid: self._validate_token(generated_tokens[rid], "generated token") for rid in expected_ids}

        finished: list[str] = []
        emitted: list[tuple[str, int]] = []
        for item in batch.items:
            request = self._requests[item.request_id]
            if item.kind is WorkKind.PREFILL:
                request.prefill_cursor += len(item.input_token_ids)
            if not item.emits_token:
                continue
            token = validated[item.request_id]
            request._generated_token_ids.append(token)
            emitted.append((item.request_id, token))
            if token in request.eos_token_ids:
                request.finish_reason = FinishReason.EOS
            elif len(request._generated_token_ids) >= request.max_new_tokens:
                request.finish_reason = FinishReason.MAX_TOKENS
            if request.finish_reason is not None:
                request.status = RequestStatus.FINISHED
                finished.append(item.request_id)
        if finished:
            gone = set(finished)
            self._running = [rid for rid in self._running if rid not in gone]
            self._finished.extend(finished)
        self._outstanding = None
        return SchedulerStepUpdate(batch.step_index, tuple(emitted), tuple(finished))

    def abort_step(self) -> SchedulerBatch:
        """Undo the outstanding batch so that the step can be tried again.  Requests admitted in
        it return to the head of the waiting queue in their order; running requests had not
        changed.  The cache side is released by the engine before this is called."""
        batch = self._outstanding
        if batch is None:
            raise RuntimeError("no scheduler batch to abort")
        admitted = batch.admitted_request_ids
        for request_id in admitted:
            request = self._requests[request_id]
            if request.prefill_cursor or request._generated_token_ids:
                raise RuntimeError(f"request {request_id!r} already has results; the step cannot be aborted")
            request.status = RequestStatus.WAITING
        gone = set(admitted)
        self._running = [rid for rid in self._running if rid not in gone]
        for request_id in reversed(admitted):
            self._waiting.appendleft(request_id)
        self._outstanding = None
        self._next_step_index = batch.step_index
        return batch

    # ------------------------------------------------------------------ validation helpers
    @classmethod
    def _validate_token_sequence(cls, values: Sequence[int], name: str) -> tuple[int, ...]:
        tokens = tuple(values)
        if not tokens:
            raise ValueError(f"{name} must not be empty")
        return tuple(cls._validate_token(token, name) for token in tokens)

    @staticmethod
    def _validate_token(value: int, name: str) -> int:
        if isinstance(value, bool) or not isinstance(value, int) or value < 0:
            raise ValueError(f"{name} must be non-negative integers")
        return value

    @classmethod
    def _normalize_eos(cls, values: int | Collection[int] | None) -> frozenset[int]:
        if values is None:
            return frozenset()
        raw = (values,) if isinstance(values, int) else tuple(values)
        return frozenset(cls._validate_token(value, "eos_token_ids") for value in raw)
