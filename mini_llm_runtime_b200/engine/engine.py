"""The synchronous engine loop: scheduler -> one model step -> sampling -> results -> release.

Entry point in the manner of the reference's ``ContinuousBatchEngine``
(src/mini_llm_runtime/engine.py:69-281): same constructor roles (scheduler, runner, admission,
clock, metrics, NVTX switch), ``submit`` and ``step``, one device-to-host copy per step (the chosen
tokens), rollback of scheduler and cache when a step fails, release of a finished request's pages
right after its results are applied.  Differences: one model call per step instead of a prefill
call plus a decode call, prompts may arrive in portions, and requests may sample with a
temperature.  ``from_model_dir`` / ``from_model`` do the assembly that the reference's runner
script does by hand (experiments/continuous_batch_engine_runner.py:227-278 there), and
``greedy_generate`` is the single-request loop of src/mini_llm_runtime/generation.py:29-117.
"""

from __future__ import annotations

import time
from collections.abc import Callable, Collection, Iterator, Sequence
from contextlib import contextmanager
from dataclasses import dataclass

import torch

from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from .admission import PagedBlockAdmissionController
from .metrics import RequestMetricsCollector
from .scheduler import (BatchingPolicy, RequestScheduler, RequestState, SchedulerBatch,
                        SchedulerStepUpdate, WorkKind)
from .step import ModelRunner, SamplingRows, StepEntry


@contextmanager
def _nvtx_range(enabled: bool, message: str) -> Iterator[None]:
    if enabled:
        torch.cuda.nvtx.range_push(message)
    try:
        yield
    finally:
        if enabled:
            torch.cuda.nvtx.range_pop()


@dataclass
class _StepAhead:
    """A decode step launched before the host had the previous step's tokens: its input ids came
    from the device.  ``request_ids`` in row order; ``host`` receives the tokens (pinned), ``event``
    marks the end of that copy."""

    request_ids: tuple[str, ...]
    tokens: torch.Tensor
    host: torch.Tensor
    event: "torch.cuda.Event | None"


@dataclass(frozen=True)
class EngineStepResult:
    batch: SchedulerBatch
    update: SchedulerStepUpdate
    released_blocks: tuple[tuple[str, dict], ...]
    started_ns: int
    tokens_ready_ns: int
    completed_ns: int


class ContinuousBatchEngine:
    def __init__(self, *, scheduler: RequestScheduler, runner: ModelRunner,
                 admission: PagedBlockAdmissionController,
                 clock_ns: Callable[[], int] = time.perf_counter_ns,
                 metrics: RequestMetricsCollector | None = None, enable_nvtx: bool = False,
                 step_ahead: bool = False) -> None:
        if admission.manager is not runner.cache:
            raise ValueError("the admission controller and the runner must share one cache manager")
        if enable_nvtx and runner.device.type != "cuda":
            raise ValueError("NVTX ranges need a CUDA engine")
        self.scheduler = scheduler
        self.runner = runner
        self.admission = admission
        self._clock_ns = clock_ns
        self.metrics = metrics or RequestMetricsCollector()
        self.enable_nvtx = enable_nvtx
        # Stepping ahead: when a step decodes only, the same requests' next decode step is launched
        # right behind it, fed on the device with the tokens it chooses, before the host reads them.
        # The host's work between two steps then runs beside the GPU instead of idling it.  What
        # step() returns does not change; a request that ends on a stop token has computed one
        # token too many, which is dropped with its pages.
        self.step_ahead = step_ahead
        self._ahead: _StepAhead | None = None
        self._token_buffers: list[torch.Tensor] = []
        self._token_buffer_cursor = 0

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
        manager = CacheManager(model.cache_needs(), page_size=block_size, num_pages=total_blocks,
                               max_requests=max_running_requests, max_tokens_per_request=max_model_len,
                               dtype=model.compute_dtype, device=model.device,
                               max_step_tokens=max_batch_tokens)
        admission = PagedBlockAdmissionController(manager)
        scheduler = RequestScheduler(max_running_requests=max_running_requests,
                                     max_batch_tokens=max_batch_tokens,
                                     max_mixed_prefill_tokens=max_mixed_prefill_tokens,
                                     admission_callback=admission.try_admit,
                                     batching_policy=batching_policy, chunked_prefill=chunked_prefill)
        return cls(scheduler=scheduler, runner=ModelRunner(model, manager), admission=admission,
                   enable_nvtx=enable_nvtx, step_ahead=step_ahead)

    @classmethod
    def from_model_dir(cls, model_dir, *, dtype="bfloat16", device="cuda:0", **options) -> "ContinuousBatchEngine":
        from ..models.factory import load_model
        _, model = load_model(model_dir, dtype, device)
        return cls.from_model(model, **options)

    @property
    def manager(self) -> CacheManager:
        return self.admission.manager

    # ------------------------------------------------------------------ requests
    def submit(self, request_id: str, prompt_token_ids: Sequence[int], *, max_new_tokens: int,
               eos_token_ids: int | Collection[int] | None = None, temperature: float = 0.0,
               seed: int = 0) -> RequestState:
        arrival_ns = self._clock_ns()
        vocab = self.runner.vocab_size
        bad = [t for t in prompt_token_ids if not isinstance(t, int) or isinstance(t, bool) or not 0 <= t < vocab]
        if bad:
            raise ValueError(f"prompt token ids must be integers in [0, {vocab}); got {bad[:5]}")
        if len(prompt_token_ids) + max_new_tokens - 1 > self.manager.max_tokens_per_request:
            raise ValueError(f"prompt + max_new_tokens - 1 = {len(prompt_token_ids) + max_new_tokens - 1} "
                             f"exceeds the engine's limit of {self.manager.max_tokens_per_request} tokens per request")
        request = self.scheduler.submit(request_id, prompt_token_ids, max_new_tokens=max_new_tokens,
                                        eos_token_ids=eos_token_ids, temperature=temperature, seed=seed)
        self.metrics.register_request(request_id, arrival_ns)
        return request

    # ------------------------------------------------------------------ one step
    @torch.inference_mode()
    def step(self) -> EngineStepResult | None:
        """Schedule and run one step; None when nothing can run."""
        started_ns = self._clock_ns()
        with _nvtx_range(self.enable_nvtx, "scheduler.schedule_step"):
            batch = self.scheduler.schedule_step()
        if batch is None:
            return None
        message = (f"engine.step:{batch.step_index}:prefill={len(batch.prefill_request_ids)}:"
                   f"decode={len(batch.decode_request_ids)}")
        with _nvtx_range(self.enable_nvtx, message):
            return self._execute_batch(batch, started_ns)

    def _execute_batch(self, batch: SchedulerBatch, started_ns: int) -> EngineStepResult:
        ahead, self._ahead = self._ahead, None
        ahead_row = {rid: row for row, rid in enumerate(ahead.request_ids)} if ahead is not None else {}
        try:
            self.metrics.require_registered(tuple(item.request_id for item in batch.items))
            # Decodes whose step is already on the GPU take their token from it; the rest is launched now.
            entries, temperatures, seeds, indices, emitting = [], [], [], [], []
            for item in batch.items:
                if item.kind is WorkKind.DECODE and item.request_id in ahead_row:
                    continue
                want = [len(item.input_token_ids) - 1] if item.emits_token else []
                entries.append(StepEntry(item.request_id, item.input_token_ids, want))
                if item.newly_admitted:
                    self.metrics.record_prefill_started(item.request_id, self._clock_ns())
                if item.emits_token:
                    request = self.scheduler.get_request(item.request_id)
                    temperatures.append(request.temperature)
                    seeds.append(request.seed)
                    indices.append(len(request.generated_token_ids))
                    emitting.append(item.request_id)
            tokens = None
            if entries:
                with _nvtx_range(self.enable_nvtx, f"model.step:tokens={sum(len(e.tokens) for e in entries)}"):
                    _, tokens = self.runner.step(entries, SamplingRows(temperatures, seeds, indices), borrow=True)
        except Exception:
            with _nvtx_range(self.enable_nvtx, "engine.rollback"):
                admitted = tuple(rid for rid in batch.admitted_request_ids
                                 if rid in self.manager.requests)
                self.admission.release_admitted(admitted)
                self.scheduler.abort_step()
            self._ahead = ahead         # its decodes are done and stay valid for the retried step
            raise

        launched = self._start_token_copy(tuple(emitting), tokens) if emitting else None
        if self.step_ahead:
            self._launch_ahead(batch, ahead, launched)

        with _nvtx_range(self.enable_nvtx, "token.d2h_sync"):
            generated: dict[str, int] = {}
            for source in (ahead, launched):
                if source is None:
                    continue
                if source.event is not None:
                    source.event.synchronize()
                values = source.host[:len(source.request_ids)].tolist()
                for rid, token in zip(source.request_ids, values, strict=True):
                    generated[rid] = int(token)
            wanted = batch.emitting_request_ids
            generated = {rid: generated[rid] for rid in wanted}     # drops rows of requests that have ended
        tokens_ready_ns = self._clock_ns()
        with _nvtx_range(self.enable_nvtx, "scheduler.apply_and_release"):
            update = self.scheduler.apply_step_results(generated)
            released = self.admission.release_finished(update.finished_request_ids)
        completed_ns = self._clock_ns()
        self.metrics.record_tokens(update.emitted_tokens, tokens_ready_ns)
        self.metrics.record_completed(update.finished_request_ids, completed_ns)
        return EngineStepResult(batch, update, tuple(released.items()), started_ns, tokens_ready_ns,
                                completed_ns)

    def _start_token_copy(self, request_ids: tuple[str, ...], tokens: torch.Tensor) -> _StepAhead:
        """Begin the device-to-host copy of a step's tokens; the caller waits on the event."""
        if tokens.device.type != "cuda":
            return _StepAhead(request_ids, tokens, tokens.to(torch.int32), None)
        if not self._token_buffers:
            size = max(64, self.scheduler.max_running_requests)
            self._token_buffers = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        host = self._token_buffers[self._token_buffer_cursor]
        self._token_buffer_cursor = (self._token_buffer_cursor + 1) % len(self._token_buffers)
        if host.numel() < tokens.numel():
            host = torch.empty(tokens.numel(), dtype=torch.int32, pin_memory=True)
        host[:tokens.numel()].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return _StepAhead(request_ids, tokens, host, event)

    def _launch_ahead(self, batch: SchedulerBatch, ahead: _StepAhead | None, launched: _StepAhead | None) -> None:
        """Launch the next decode step of this batch's requests behind the current one, if the
        current one decodes only, all of its tokens lie in one device tensor in the batch's order,
        and none of its requests reaches its token limit with this step."""
        rids = tuple(item.request_id for item in batch.items)
        if not batch.items or any(item.kind is not WorkKind.DECODE for item in batch.items):
            return
        if ahead is not None and launched is None and ahead.request_ids == rids:
            source = ahead
        elif ahead is None and launched is not None and launched.request_ids == rids:
            source = launched
        else:
            return
        requests = [self.scheduler.get_request(rid) for rid in rids]
        if any(len(r.generated_token_ids) + 1 >= r.max_new_tokens for r in requests):
            return
        entries = [StepEntry(rid, [0], [0]) for rid in rids]
        sampling = SamplingRows([r.temperature for r in requests], [r.seed for r in requests],
                                [len(r.generated_token_ids) + 1 for r in requests])
        try:
            with _nvtx_range(self.enable_nvtx, f"model.step_ahead:tokens={len(entries)}"):
                _, tokens = self.runner.step(entries, sampling, borrow=True, feed=source.tokens)
        except Exception:
            return          # nothing was launched and the cache is as before: go on step by step
        self._ahead = self._start_token_copy(rids, tokens)

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
        first = len(self.scheduler.finished_request_ids) + len(self.scheduler.running_request_ids) \
            + len(self.scheduler.waiting_request_ids)
        ids = [f"generate-{first + i}" for i in range(len(prompts))]
        for i, (request_id, prompt) in enumerate(zip(ids, prompts)):
            self.submit(request_id, list(prompt), max_new_tokens=max_new_tokens,
                        eos_token_ids=eos_token_ids, temperature=temperature, seed=seed + i)
        self.run()
        return [list(self.scheduler.get_request(request_id).generated_token_ids) for request_id in ids]


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
            token = int(torch.argmax(logits[0]))
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
