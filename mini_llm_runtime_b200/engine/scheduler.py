"""The request scheduler: who runs in the next step, with how many tokens.

It keeps the rules of the reference's ``RequestScheduler``
(src/mini_llm_runtime/scheduler.py:205-288 for scheduling, :290-373 for results and abort, and
block_admission.py:35-93 for page admission) on a data model of its own:

* every request that has consumed its prompt decodes once per step, before anything else is
  considered (decode first);
* prompts that are already under way get their next portion, in arrival order;
* waiting prompts are admitted from the head of the queue only; the first one that does not fit
  (no free place, no token budget left, or the page gate says no) stops admission for this step and
  is never overtaken (strict FIFO, head-of-line blocking);
* a step that began with running requests may spend at most ``max_mixed_prefill_tokens`` on prompt
  tokens, so that decodes are not starved by long prompts;
* ``STATIC`` batching admits only while nothing is running (a cohort drains before the next);
* a stop token ends a request even on the step that reaches its token limit;
* scheduling and results alternate; an aborted step returns the requests it admitted to the head of
  the queue in their order and the step keeps its index.

New here is the *portion*: the reference refuses prompts longer than the token budget
(scheduler.py:181-185).  Here such a prompt is admitted with as many tokens as fit, stays running
while it consumes further portions, and emits its first token with its last portion.
``chunked_prefill=False`` restores the reference's whole-prompt rule.

Pages.  The scheduler owns admission: before a request leaves the queue it asks the *gate* (the
cache manager, through ``CacheGate``) for a slot and a promise of the pages of the request's whole
life, and it gives both back when the request finishes, is aborted or fails.  When pages run out
the decision is the reference's: the head of the queue waits, and everything behind it, until a
finished request frees pages; nothing is preempted, swapped or recomputed.  Because the promise
covers a request's whole life, a running request never finds the pool empty.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Collection, Mapping, Sequence
from dataclasses import dataclass, field
from enum import Enum
from typing import Protocol

import numpy as np

from ..sampling import GREEDY, SamplingParams


class RequestStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(str, Enum):
    EOS = "eos"
    MAX_TOKENS = "max_tokens"
    ERROR = "error"            # the step that ran it reported a device error; its output is cut short


class WorkKind(str, Enum):
    PREFILL = "prefill"
    DECODE = "decode"


class BatchingPolicy(str, Enum):
    """CONTINUOUS refills free places while others still run; STATIC waits for the cohort to drain."""

    CONTINUOUS = "continuous"
    STATIC = "static"


def _token(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ValueError(f"{what} must be non-negative integers, got {value!r}")
    return value


@dataclass
class Request:
    """One request as the scheduler sees it.  It holds no device memory; ``slot`` names the place
    the cache manager gave it while it runs."""

    request_id: str
    prompt: tuple[int, ...]
    max_new_tokens: int
    stop_tokens: frozenset[int]
    sampling: SamplingParams
    order: int                                  # arrival number: the queue's order
    status: RequestStatus = RequestStatus.WAITING
    cursor: int = 0                             # prompt tokens consumed by applied steps
    output: list[int] = field(default_factory=list, repr=False)
    finish_reason: FinishReason | None = None
    slot: int | None = None
    _prompt_array: "np.ndarray | None" = field(default=None, repr=False, compare=False)

    @property
    def prompt_token_ids(self) -> tuple[int, ...]:
        return self.prompt

    def prompt_span(self, start: int, count: int) -> "np.ndarray":
        """``count`` prompt tokens from ``start`` as a view of one int32 array (made once: the step
        function takes arrays as they are, while a tuple of thousands of integers costs it a
        conversion per portion)."""
        if self._prompt_array is None:
            self._prompt_array = np.asarray(self.prompt, dtype=np.int32)
        return self._prompt_array[start:start + count]

    @property
    def generated_token_ids(self) -> tuple[int, ...]:
        return tuple(self.output)

    @property
    def prompt_done(self) -> bool:
        return self.cursor >= len(self.prompt)

    @property
    def lifetime_tokens(self) -> int:
        """Most tokens the cache ever holds for it: the last generated token is never fed back
        (reference: scheduler.py:52-55)."""
        return len(self.prompt) + self.max_new_tokens - 1

    @property
    def temperature(self) -> float:
        return self.sampling.temperature

    @property
    def seed(self) -> int:
        return self.sampling.seed


@dataclass(frozen=True)
class WorkItem:
    """One request's input to the model in one step."""

    request_id: str
    kind: WorkKind
    tokens: tuple[int, ...]
    emits: bool = True          # False for a prompt portion that is not the last
    admitted: bool = False      # the request left the queue in this step
    slot: int | None = None


@dataclass(frozen=True)
class StepPlan:
    index: int
    items: tuple[WorkItem, ...]

    @property
    def token_count(self) -> int:
        return sum(len(item.tokens) for item in self.items)

    def ids(self, *, kind: WorkKind | None = None, admitted: bool | None = None,
            emits: bool | None = None) -> tuple[str, ...]:
        return tuple(item.request_id for item in self.items
                     if (kind is None or item.kind is kind)
                     and (admitted is None or item.admitted == admitted)
                     and (emits is None or item.emits == emits))

    @property
    def prefill_request_ids(self) -> tuple[str, ...]:
        return self.ids(kind=WorkKind.PREFILL)

    @property
    def decode_request_ids(self) -> tuple[str, ...]:
        return self.ids(kind=WorkKind.DECODE)

    @property
    def admitted_request_ids(self) -> tuple[str, ...]:
        return self.ids(admitted=True)

    @property
    def emitting_request_ids(self) -> tuple[str, ...]:
        return self.ids(emits=True)

    @property
    def decode_only(self) -> bool:
        return all(item.kind is WorkKind.DECODE for item in self.items)


@dataclass(frozen=True)
class StepOutcome:
    index: int
    emitted_tokens: tuple[tuple[str, int], ...]
    finished_request_ids: tuple[str, ...]
    freed: Mapping[str, object] = field(default_factory=dict)    # what the gate gave back per finished request


class Gate(Protocol):
    """Where admitted requests get their resources.  ``admit`` answers with the request's slot, or
    None having changed nothing; ``release`` gives everything back."""

    def admit(self, request: Request) -> int | None: ...

    def release(self, request_id: str) -> object: ...


class CacheGate:
    """The cache manager as the scheduler's gate: a slot and a promise of pages for the request's
    whole life (prompt + max_new_tokens - 1 tokens), sampling parameters into the slot's record."""

    def __init__(self, cache) -> None:
        self.cache = cache

    def admit(self, request: Request) -> int | None:
        held = self.cache.create_request(request.request_id, lifetime_tokens=request.lifetime_tokens,
                                         temperature=request.sampling.temperature, seed=request.sampling.seed)
        return None if held is None else held.slot

    def release(self, request_id: str):
        return self.cache.release(request_id) if request_id in self.cache.requests else {}


class _Budget:
    """What is left of a step's limits while the step is put together."""

    def __init__(self, tokens: int, prompt_tokens: int | None) -> None:
        self.tokens = tokens
        self.prompt_tokens = prompt_tokens      # None: prompt tokens are limited by ``tokens`` only

    def room_for_prompt(self) -> int:
        return self.tokens if self.prompt_tokens is None else min(self.tokens, self.prompt_tokens)

    def spend(self, count: int, *, prompt: bool) -> None:
        self.tokens -= count
        if prompt and self.prompt_tokens is not None:
            self.prompt_tokens -= count


class RequestScheduler:
    def __init__(self, *, max_running_requests: int, max_batch_tokens: int,
                 max_mixed_prefill_tokens: int | None = None, gate: Gate | None = None,
                 batching_policy: BatchingPolicy = BatchingPolicy.CONTINUOUS,
                 chunked_prefill: bool = True) -> None:
        for name, value in (("max_running_requests", max_running_requests), ("max_batch_tokens", max_batch_tokens)):
            if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if max_running_requests > max_batch_tokens:
            raise ValueError("max_running_requests must not exceed max_batch_tokens: every running request "
                             "needs one token of the budget to decode")
        if max_mixed_prefill_tokens is not None and (
                isinstance(max_mixed_prefill_tokens, bool) or not isinstance(max_mixed_prefill_tokens, int)
                or max_mixed_prefill_tokens <= 0):
            raise ValueError("max_mixed_prefill_tokens must be a positive integer or None")
        if not isinstance(batching_policy, BatchingPolicy):
            raise ValueError("batching_policy must be a BatchingPolicy")
        self.max_running_requests = max_running_requests
        self.max_batch_tokens = max_batch_tokens
        self.max_mixed_prefill_tokens = max_mixed_prefill_tokens
        self.batching_policy = batching_policy
        self.chunked_prefill = chunked_prefill
        self.gate = gate
        self._by_id: dict[str, Request] = {}
        self._queue: deque[Request] = deque()           # waiting, arrival order
        self._live: dict[str, Request] = {}             # running, admission order
        self._done: list[str] = []
        self._arrivals = 0
        self._step_index = 0
        self._plan: StepPlan | None = None

    # ------------------------------------------------------------------ what is where
    @property
    def waiting_request_ids(self) -> tuple[str, ...]:
        return tuple(request.request_id for request in self._queue)

    @property
    def running_request_ids(self) -> tuple[str, ...]:
        return tuple(self._live)

    @property
    def finished_request_ids(self) -> tuple[str, ...]:
        return tuple(self._done)

    @property
    def outstanding_plan(self) -> StepPlan | None:
        return self._plan

    @property
    def has_unfinished_requests(self) -> bool:
        return bool(self._queue or self._live or self._plan)

    def get_request(self, request_id: str) -> Request:
        try:
            return self._by_id[request_id]
        except KeyError:
            raise KeyError(f"unknown request_id={request_id!r}") from None

    # ------------------------------------------------------------------ arrival
    def submit(self, request_id: str, prompt_token_ids: Sequence[int], *, max_new_tokens: int,
               eos_token_ids: int | Collection[int] | None = None, temperature: float = 0.0,
               seed: int = 0, sampling: SamplingParams | None = None) -> Request:
        """Queue a request; allowed at any time, also while a plan is outstanding."""
        if not request_id:
            raise ValueError("request_id must not be empty")
        if request_id in self._by_id:
            raise ValueError(f"request_id={request_id!r} already exists")
        prompt = tuple(_token(t, "prompt_token_ids") for t in prompt_token_ids)
        if not prompt:
            raise ValueError("prompt_token_ids must not be empty")
        if not self.chunked_prefill and len(prompt) > self.max_batch_tokens:
            raise ValueError(f"prompt length={len(prompt)} exceeds max_batch_tokens={self.max_batch_tokens} "
                             "and chunked prefill is off")
        if isinstance(max_new_tokens, bool) or not isinstance(max_new_tokens, int) or max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be a positive integer")
        if eos_token_ids is None:
            stop = frozenset()
        else:
            stop = frozenset(_token(t, "eos_token_ids")
                             for t in ((eos_token_ids,) if isinstance(eos_token_ids, int) else eos_token_ids))
        if sampling is None:
            sampling = SamplingParams(temperature, seed) if (temperature or seed) else GREEDY
        request = Request(request_id, prompt, max_new_tokens, stop, sampling, order=self._arrivals)
        self._arrivals += 1
        self._by_id[request_id] = request
        self._queue.append(request)
        return request

    # ------------------------------------------------------------------ the next step
    def schedule_step(self) -> StepPlan | None:
        if self._plan is not None:
            raise RuntimeError("the previous plan has been neither applied nor aborted")
        if not self._live and not self._queue:
            return None
        began_with_running = bool(self._live)
        budget = _Budget(self.max_batch_tokens,
                         self.max_mixed_prefill_tokens if began_with_running else None)
        items: list[WorkItem] = []

        for request in self._live.values():                 # 1. decodes
            if request.prompt_done:
                if not request.output:
                    raise RuntimeError(f"running request {request.request_id!r} has consumed its prompt "
                                       "but has no token to feed back")
                items.append(WorkItem(request.request_id, WorkKind.DECODE, (request.output[-1],), slot=request.slot))
                budget.spend(1, prompt=False)

        for request in self._live.values():                 # 2. prompts under way
            if request.prompt_done:
                continue
            room = budget.room_for_prompt()
            if room <= 0:
                break
            items.append(self._portion(request, room, admitted=False))
            budget.spend(len(items[-1].tokens), prompt=True)

        may_admit = self.batching_policy is BatchingPolicy.CONTINUOUS or not began_with_running
        while may_admit and self._queue and len(self._live) < self.max_running_requests:   # 3. admission
            request = self._queue[0]
            room = budget.room_for_prompt()
            if room <= 0 or (not self.chunked_prefill and len(request.prompt) > room):
                break
            if self.gate is not None:
                slot = self.gate.admit(request)
                if slot is None:
                    break
                request.slot = slot
            self._queue.popleft()
            request.status = RequestStatus.RUNNING
            self._live[request.request_id] = request
            items.append(self._portion(request, room, admitted=True))
            budget.spend(len(items[-1].tokens), prompt=True)

        if not items:
            return None
        self._plan = StepPlan(self._step_index, tuple(items))
        self._step_index += 1
        return self._plan

    @staticmethod
    def _portion(request: Request, room: int, *, admitted: bool) -> WorkItem:
        left = len(request.prompt) - request.cursor
        count = min(left, room)
        tokens = request.prompt[request.cursor:request.cursor + count]
        return WorkItem(request.request_id, WorkKind.PREFILL, tokens, emits=count == left, admitted=admitted,
                        slot=request.slot)

    # ------------------------------------------------------------------ what the step produced
    def apply_step_results(self, generated_tokens: Mapping[str, int]) -> StepOutcome:
        """One token for every item that emits one.  Everything is checked before anything changes."""
        plan = self._plan
        if plan is None:
            raise RuntimeError("no plan is waiting for results")
        expected = plan.emitting_request_ids
        if len(generated_tokens) != len(expected) or set(generated_tokens) != set(expected):
            missing = sorted(set(expected) - set(generated_tokens))
            extra = sorted(set(generated_tokens) - set(expected))
            raise ValueError(f"step results do not match the plan: missing={missing}, extra={extra}")
        checked = {rid: _token(generated_tokens[rid], "generated tokens") for rid in expected}

        emitted: list[tuple[str, int]] = []
        finished: list[str] = []
        for item in plan.items:
            request = self._by_id[item.request_id]
            if item.kind is WorkKind.PREFILL:
                request.cursor += len(item.tokens)
            if not item.emits:
                continue
            token = checked[item.request_id]
            request.output.append(token)
            emitted.append((item.request_id, token))
            if token in request.stop_tokens:
                request.finish_reason = FinishReason.EOS
            elif len(request.output) >= request.max_new_tokens:
                request.finish_reason = FinishReason.MAX_TOKENS
            if request.finish_reason is not None:
                finished.append(item.request_id)
        freed = {rid: self._retire(self._by_id[rid]) for rid in finished}
        self._plan = None
        return StepOutcome(plan.index, tuple(emitted), tuple(finished), freed)

    def _retire(self, request: Request):
        request.status = RequestStatus.FINISHED
        self._live.pop(request.request_id, None)
        self._done.append(request.request_id)
        slot, request.slot = request.slot, None
        return self.gate.release(request.request_id) if self.gate is not None and slot is not None else {}

    def abort_step(self) -> StepPlan:
        """Take the outstanding plan back so that the step can be tried again.  Requests it admitted
        give their slot and pages back and return to the head of the queue in their order; the
        others had not changed.  The step keeps its index."""
        plan = self._plan
        if plan is None:
            raise RuntimeError("no plan to abort")
        returned = [self._by_id[rid] for rid in plan.admitted_request_ids]
        for request in returned:
            if request.cursor or request.output:
                raise RuntimeError(f"request {request.request_id!r} already has results; its step cannot be aborted")
        for request in reversed(returned):
            del self._live[request.request_id]
            if self.gate is not None and request.slot is not None:
                self.gate.release(request.request_id)
            request.slot = None
            request.status = RequestStatus.WAITING
            self._queue.appendleft(request)
        self._plan = None
        self._step_index = plan.index
        return plan

    def fail_requests(self, request_ids: Collection[str]) -> tuple[str, ...]:
        """End the named requests with ``FinishReason.ERROR`` wherever they are, give their resources
        back and drop the outstanding plan.  For results that cannot be trusted (a device error)."""
        failed = []
        for request_id in request_ids:
            request = self._by_id[request_id]
            if request.status is RequestStatus.FINISHED:
                continue
            if request.status is RequestStatus.WAITING:
                self._queue.remove(request)
            request.finish_reason = FinishReason.ERROR
            self._retire(request)
            failed.append(request_id)
        self._plan = None
        return tuple(failed)
