"""The synchronous engine loop: plan a step, run it as one model call, sample on the device, read
the tokens, apply them, free what finished.

An entry point in the manner of the reference's ``ContinuousBatchEngine``
(src/mini_llm_runtime/engine.py:69-281): ``submit`` and ``step``, one device-to-host copy per step
(the chosen tokens), scheduler and cache rolled back when a step fails, a finished request's pages
free right after its results are applied, optional NVTX ranges under the reference's names.
Differences: one model call per step where the reference makes a prefill call and a decode call;
prompts may arrive in portions; requests may sample with a temperature; page admission is part of
the scheduler (its gate), so the constructor takes no admission controller; and a step of decoded
tokens sends the device nothing but the slots of its requests, because positions, last tokens and
sampling state live in the requests' slot records.  ``from_model_dir`` / ``from_model`` do the
assembly that the reference's runner script does by hand
(experiments/continuous_batch_engine_runner.py:227-278 there), and ``greedy_generate`` is the
single-request loop of src/mini_llm_runtime/generation.py:29-117.
"""

from __future__ import annotations

import contextlib
import time
from collections.abc import Callable, Collection, Sequence
from dataclasses import dataclass

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from ..sampling import SamplingParams
from .metrics import RequestMetricsCollector
from .scheduler import BatchingPolicy, CacheGate, Request, RequestScheduler, StepOutcome, StepPlan, WorkKind
from .step import ModelRunner, StepEntry


@dataclass
class _TokensInFlight:
    """The tokens of a launched step on their way to the host: ``request_ids`` in row order, ``host``
    the pinned destination, ``event`` the end of the copy (None when nothing is asynchronous)."""

    request_ids: tuple[str, ...]
    host: torch.Tensor
    event: "torch.cuda.Event | None"

    def wait(self) -> dict[str, int]:
        if self.event is not None:
            self.event.synchronize()
        return dict(zip(self.request_ids, self.host[:len(self.request_ids)].tolist(), strict=True))


@dataclass(frozen=True)
class EngineStepResult:
    """One engine step: what was planned, what came out, and when (nanoseconds of the engine's clock)."""

    plan: StepPlan
    outcome: StepOutcome
    started_ns: int
    tokens_ready_ns: int
    completed_ns: int

    @property
    def freed(self):
        return self.outcome.freed


class ContinuousBatchEngine:
    def __init__(self, *, scheduler: RequestScheduler, runner: ModelRunner,
                 clock_ns: Callable[[], int] = time.perf_counter_ns,
                 metrics: RequestMetricsCollector | None = None, enable_nvtx: bool = False,
                 step_ahead: bool = False) -> None:
        gate = scheduler.gate
        if not isinstance(gate, CacheGate) or gate.cache is not runner.cache:
            raise ValueError("the scheduler's gate must be a CacheGate on the runner's cache manager")
        if enable_nvtx and runner.device.type != "cuda":
            raise ValueError("NVTX ranges need a CUDA engine")
        self.scheduler = scheduler
        self.runner = runner
        self._clock_ns = clock_ns
        self.metrics = metrics or RequestMetricsCollector()
        self.enable_nvtx = enable_nvtx
        # Stepping ahead: when a step decodes only, the same requests' next decode step is launched
        # right behind it, before the host has read the tokens: the device takes each request's input
        # from its slot record, where the sampling kernel has just stored it.  The host's work between
        # two steps then runs beside the GPU instead of idling it.  What step() returns does not
        # change; a request that ends on a stop token has computed one token too many, which is
        # dropped with its pages.
        self.step_ahead = step_ahead
        self._ahead: _TokensInFlight | None = None
        self._token_buffers: list[torch.Tensor] = []
        self._next_buffer = 0

    # ------------------------------------------------------------------ assembly
    @classmethod
    def from_model(cls, model: DecoderModel, *, block_size: int = 16, total_blocks: int | None = None,
                   max_running_requests: int = 8, max_batch_tokens: int = 2048,
                   max_mixed_prefill_tokens: int | None = None, max_model_len: int | None = None,
                   batching_policy: BatchingPolicy = BatchingPolicy.CONTINUOUS,
                   chunked_prefill: bool = True, enable_nvtx: bool = False,
                   step_ahead: bool = False) -> "ContinuousBatchEngine":
        max_model_len = min(max_model_len or model.spec.max_positions, model.spec.max_positions)
        if total_blocks is None:
            total_blocks = max_running_requests * -(-max_model_len // block_size)
        cache = CacheManager(model.cache_needs(), page_size=block_size, num_pages=total_blocks,
                             max_requests=max_running_requests, max_tokens_per_request=max_model_len,
                             dtype=model.compute_dtype, device=model.device, max_step_tokens=max_batch_tokens)
        scheduler = RequestScheduler(max_running_requests=max_running_requests, max_batch_tokens=max_batch_tokens,
                                     max_mixed_prefill_tokens=max_mixed_prefill_tokens, gate=CacheGate(cache),
                                     batching_policy=batching_policy, chunked_prefill=chunked_prefill)
        return cls(scheduler=scheduler, runner=ModelRunner(model, cache), enable_nvtx=enable_nvtx,
                   step_ahead=step_ahead)

    @classmethod
    def from_model_dir(cls, model_dir, *, dtype="bfloat16", device="cuda:0", **options) -> "ContinuousBatchEngine":
        from ..models.factory import load_model
        _, model = load_model(model_dir, dtype, device)
        return cls.from_model(model, **options)

    @property
    def manager(self) -> CacheManager:
        return self.runner.cache

    def _range(self, message: str):
        """An NVTX range around a phase of the step when tracing is on (names as in the reference:
        engine.py:158-168,191-195,233-236,251,257,267)."""
        return torch.cuda.nvtx.range(message) if self.enable_nvtx else contextlib.nullcontext()

    # ------------------------------------------------------------------ requests
    def submit(self, request_id: str, prompt_token_ids: Sequence[int], *, max_new_tokens: int,
               eos_token_ids: int | Collection[int] | None = None, temperature: float = 0.0,
               seed: int = 0) -> Request:
        arrival_ns = self._clock_ns()
        vocab = self.runner.vocab_size
        outside = [t for t in prompt_token_ids if not isinstance(t, int) or isinstance(t, bool) or not 0 <= t < vocab]
        if outside:
            raise ValueError(f"prompt token ids must be integers in [0, {vocab}); got {outside[:5]}")
        longest = len(prompt_token_ids) + max_new_tokens - 1
        if longest > self.manager.max_tokens_per_request:
            raise ValueError(f"prompt + max_new_tokens - 1 = {longest} exceeds the engine's limit of "
                             f"{self.manager.max_tokens_per_request} tokens per request")
        request = self.scheduler.submit(request_id, prompt_token_ids, max_new_tokens=max_new_tokens,
                                        eos_token_ids=eos_token_ids,
                                        sampling=SamplingParams(temperature, seed))
        self.metrics.register_request(request_id, arrival_ns)
        return request

    # ------------------------------------------------------------------ one step
    @torch.inference_mode()
    def step(self) -> EngineStepResult | None:
        """Plan and run one step; None when nothing can run."""
        started_ns = self._clock_ns()
        with self._range("scheduler.schedule_step"):
            plan = self.scheduler.schedule_step()
        if plan is None:
            return None
        with self._range(f"engine.step:{plan.index}:prefill={len(plan.prefill_request_ids)}:"
                         f"decode={len(plan.decode_request_ids)}"):
            return self._run(plan, started_ns)

    def _run(self, plan: StepPlan, started_ns: int) -> EngineStepResult:
        ahead, self._ahead = self._ahead, None
        covered = set(ahead.request_ids) if ahead is not None else set()
        try:
            self.metrics.require_registered(tuple(item.request_id for item in plan.items))
            # Decodes whose step is already on the GPU take their token from it; the rest is launched now.
            entries, emitting = [], []
            for item in plan.items:
                if item.kind is WorkKind.DECODE and item.request_id in covered:
                    continue
                tokens = item.tokens
                if item.kind is not WorkKind.DECODE and len(tokens) > 16:
                    request = self.scheduler.get_request(item.request_id)     # a prompt portion: starts at the cursor
                    tokens = request.prompt_span(request.cursor, len(tokens))
                entries.append(StepEntry(item.request_id, tokens, [len(tokens) - 1] if item.emits else []))
                if item.admitted:
                    self.metrics.record_prefill_started(item.request_id, self._clock_ns())
                if item.emits:
                    emitting.append(item.request_id)
            launched = None
            if entries:
                with self._range(f"model.step:tokens={sum(len(e.tokens) for e in entries)}"):
                    # a step of decodes takes its inputs from the slot records (the tokens sampled last)
                    decodes_only = all(item.kind is WorkKind.DECODE for item in plan.items)
                    _, tokens = self.runner.step(entries, sample=True, borrow=True, feed=decodes_only)
                if emitting:
                    launched = self._start_token_copy(tuple(emitting), tokens)
        except Exception:
            with self._range("engine.rollback"):
                self.scheduler.abort_step()      # the requests it admitted give slot and pages back
            self._ahead = ahead                  # its decodes are done and stay valid for the retried step
            raise

        if self.step_ahead:
            self._launch_ahead(plan, ahead, launched)

        with self._range("token.d2h_sync"):
            generated: dict[str, int] = {}
            for source in (ahead, launched):
                if source is not None:
                    generated.update(source.wait())
            try:
                self.runner.check_device()
            except ops.KernelError:
                self._give_up_after_device_error(plan)
                raise
            generated = {rid: generated[rid] for rid in plan.emitting_request_ids}   # drops rows of ended requests
        tokens_ready_ns = self._clock_ns()
        with self._range("scheduler.apply_and_release"):
            outcome = self.scheduler.apply_step_results(generated)
        completed_ns = self._clock_ns()
        self.metrics.record_tokens(outcome.emitted_tokens, tokens_ready_ns)
        self.metrics.record_completed(outcome.finished_request_ids, completed_ns)
        return EngineStepResult(plan, outcome, started_ns, tokens_ready_ns, completed_ns)

    def _give_up_after_device_error(self, plan: StepPlan) -> None:
        """A kernel reported that a bounded wait ran out: nothing computed since the last check can
        be trusted, and the cache already holds those steps' keys and values.  The requests of the
        step (and of the step launched ahead of it) end with ``FinishReason.ERROR`` and give their
        pages back; waiting requests and the engine itself stay usable."""
        with self._range("engine.rollback"):
            touched = [item.request_id for item in plan.items]
            if self._ahead is not None:
                touched += [rid for rid in self._ahead.request_ids if rid not in touched]
                self._ahead.wait()
                self._ahead = None
            failed = self.scheduler.fail_requests(touched)
            self.metrics.record_completed(failed, self._clock_ns())

    def _start_token_copy(self, request_ids: tuple[str, ...], tokens: torch.Tensor) -> _TokensInFlight:
        """Begin the device-to-host copy of a step's tokens; the caller waits on the event."""
        if tokens.device.type != "cuda":
            return _TokensInFlight(request_ids, tokens.to(torch.int32), None)
        if not self._token_buffers:
            size = max(64, self.scheduler.max_running_requests)
            self._token_buffers = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        host = self._token_buffers[self._next_buffer]
        self._next_buffer = (self._next_buffer + 1) % len(self._token_buffers)
        if host.numel() < tokens.numel():
            host = torch.empty(tokens.numel(), dtype=torch.int32, pin_memory=True)
        host[:tokens.numel()].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return _TokensInFlight(request_ids, host, event)

    def _launch_ahead(self, plan: StepPlan, ahead: _TokensInFlight | None, launched: _TokensInFlight | None) -> None:
        """Launch the next decode step of this plan's requests behind the current one, if the
        current one decodes only, was launched (or had been launched ahead) as one step in the plan's
        order, and none of its requests reaches its token limit with this step."""
        if not plan.items or not plan.decode_only:
            return
        request_ids = tuple(item.request_id for item in plan.items)
        current = ahead if launched is None else (launched if ahead is None else None)
        if current is None or current.request_ids != request_ids:
            return
        requests = [self.scheduler.get_request(rid) for rid in request_ids]
        if any(len(request.output) + 1 >= request.max_new_tokens for request in requests):
            return
        entries = [StepEntry(rid, [0], [0]) for rid in request_ids]
        try:
            with self._range(f"model.step_ahead:tokens={len(entries)}"):
                _, tokens = self.runner.step(entries, sample=True, borrow=True, feed=True)
        except Exception:
            return          # nothing was launched and the cache is as before: go on step by step
        self._ahead = self._start_token_copy(request_ids, tokens)

    # ------------------------------------------------------------------ conveniences
    def run(self) -> list[EngineStepResult]:
        """Step until every submitted request has finished."""
        results = []
        while self.scheduler.has_unfinished_requests:
            result = self.step()
            if result is None:
                raise RuntimeError("requests are waiting but nothing can be scheduled")
            results.append(result)
        return results

    def generate(self, prompts: Sequence[Sequence[int]], *, max_new_tokens: int,
                 eos_token_ids: int | Collection[int] | None = None, temperature: float = 0.0,
                 seed: int = 0) -> list[list[int]]:
        """Token ids in, generated token ids out, for a list of prompts (host lists both ways)."""
        scheduler = self.scheduler
        first = (len(scheduler.finished_request_ids) + len(scheduler.running_request_ids)
                 + len(scheduler.waiting_request_ids))
        ids = [f"generate-{first + i}" for i in range(len(prompts))]
        for i, (request_id, prompt) in enumerate(zip(ids, prompts)):
            self.submit(request_id, list(prompt), max_new_tokens=max_new_tokens,
                        eos_token_ids=eos_token_ids, temperature=temperature, seed=seed + i)
        self.run()
        return [list(scheduler.get_request(request_id).generated_token_ids) for request_id in ids]


@dataclass(frozen=True)
class GreedyGenerationOutput:
    generated_token_ids: list[int]
    stopped_by_eos: bool
    prefill_tokens: int
    decode_steps: int
    cache_length: int
    step_logits: tuple[torch.Tensor, ...] | None = None


@torch.inference_mode()
def greedy_generate(runner: ModelRunner, input_ids: Sequence[int], *, max_new_tokens: int,
                    eos_token_ids: int | Collection[int] | None = None,
                    return_step_logits: bool = False, request_id: str = "greedy") -> GreedyGenerationOutput:
    """One prompt, one prefill step, then one-token steps (reference: generation.py:29-117).  EOS
    is tested before the token would be fed back; N tokens need N-1 decode steps and leave
    prompt + N - 1 tokens in the cache, which is given back at the end."""
    prompt = [int(t) for t in input_ids]
    if not prompt:
        raise ValueError("greedy_generate needs a non-empty prompt")
    if max_new_tokens <= 0:
        raise ValueError("max_new_tokens must be > 0")
    if eos_token_ids is None:
        eos = frozenset()
    else:
        eos = frozenset([eos_token_ids] if isinstance(eos_token_ids, int) else [int(t) for t in eos_token_ids])
    invalid = sorted(t for t in eos if not 0 <= t < runner.vocab_size)
    if invalid:
        raise ValueError(f"EOS token ids outside the vocabulary: {invalid}")
    if len(prompt) + max_new_tokens - 1 > min(runner.max_positions, runner.cache.max_tokens_per_request):
        raise ValueError("prompt_length + max_new_tokens - 1 exceeds the model's or the cache's limit")
    runner.cache.create_request(request_id)
    generated: list[int] = []
    captured: list[torch.Tensor] = []
    stopped = False
    decode_steps = 0
    try:
        logits = runner.step([StepEntry(request_id, prompt, [len(prompt) - 1])])
        for index in range(max_new_tokens):
            if return_step_logits:
                captured.append(logits[0].clone())
            token = int(torch.argmax(logits[0]))     # the host waits for the step here
            runner.check_device()
            generated.append(token)
            stopped = token in eos
            if stopped or index == max_new_tokens - 1:
                break
            logits = runner.step([StepEntry(request_id, [token], [0])])
            decode_steps += 1
        cache_length = runner.cache.get(request_id).committed
    finally:
        runner.cache.release(request_id)
    return GreedyGenerationOutput(generated, stopped, len(prompt), decode_steps, cache_length,
                                  tuple(captured) if return_step_logits else None)
