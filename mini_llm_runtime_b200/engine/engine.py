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
                 metrics: RequestMetricsCollector | None = None, enable_nvtx: bool = False) -> None:
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

    # ------------------------------------------------------------------ assembly
    @classmethod
    def from_model(cls, model: DecoderModel, *, block_size: int = 16, total_blocks: int | None = None,
                   max_running_requests: int = 8, max_batch_tokens: int = 2048,
                   max_mixed_prefill_tokens: int | None = None, max_model_len: int | None = None,
                   batching_policy: BatchingPolicy = BatchingPolicy.CONTINUOUS,
                   chunked_prefill: bool = True, enable_nvtx: bool = False) -> "ContinuousBatchEngine":
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
                   enable_nvtx=enable_nvtx)

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
        try:
            self.metrics.require_registered(tuple(item.request_id for item in batch.items))
            entries, temperatures, seeds, indices, emitting = [], [], [], [], []
            for item in batch.items:
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
            with _nvtx_range(self.enable_nvtx, f"model.step:tokens={batch.token_count}"):
                _, tokens = self.runner.step(entries, SamplingRows(temperatures, seeds, indices), borrow=True)
        except Exception:
            with _nvtx_range(self.enable_nvtx, "engine.rollback"):
                admitted = tuple(rid for rid in batch.admitted_request_ids
                                 if rid in self.manager.requests)
                self.admission.release_admitted(admitted)
                self.scheduler.abort_step()
            raise

        with _nvtx_range(self.enable_nvtx, "token.d2h_sync"):
            host_tokens = tokens.cpu().tolist() if emitting else []
        tokens_ready_ns = self._clock_ns()
        generated = {rid: int(token) for rid, token in zip(emitting, host_tokens, strict=True)}
        with _nvtx_range(self.enable_nvtx, "scheduler.apply_and_release"):
            update = self.scheduler.apply_step_results(generated)
            released = self.admission.release_finished(update.finished_request_ids)
        completed_ns = self._clock_ns()
        self.metrics.record_tokens(update.emitted_tokens, tokens_ready_ns)
        self.metrics.record_completed(update.finished_request_ids, completed_ns)
        return EngineStepResult(batch, update, tuple(released.items()), started_ns, tokens_ready_ns,
                                completed_ns)

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
