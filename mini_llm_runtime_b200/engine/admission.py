"""Bridge between the scheduler and the cache manager: a request is admitted only if the pages of
its whole life can be promised to it.

Same policy as the reference's ``PagedBlockAdmissionController``
(src/mini_llm_runtime/block_admission.py:18-93): pages for prompt + max_new_tokens - 1 tokens,
rounded up to whole pages, are set aside at admission; too few left means "not now" with no side
effect; more than the pool will ever hold is an error.  The difference: the reference takes the
physical blocks at once, here they are counted as promised and taken as tokens arrive, which also
covers groups of layers with a sliding window, whose need is bounded by the window.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..cache.manager import CacheManager
from .scheduler import RequestState


@dataclass(frozen=True)
class BlockReservation:
    request_id: str
    max_cache_tokens: int
    block_counts: tuple[int, ...]     # pages promised per cache group


class PagedBlockAdmissionController:
    def __init__(self, manager: CacheManager) -> None:
        self.manager = manager
        self._reservations: dict[str, BlockReservation] = {}

    @property
    def reservations(self) -> tuple[BlockReservation, ...]:
        return tuple(self._reservations.values())

    def reservation_for(self, request_id: str) -> BlockReservation:
        try:
            return self._reservations[request_id]
        except KeyError:
            raise KeyError(f"request {request_id!r} has no page reservation") from None

    def try_admit(self, request: RequestState) -> bool:
        """True: the request has a cache entry and its pages are promised.  False: nothing changed.
        Raises ValueError when the request could never fit."""
        if request.request_id in self._reservations:
            raise RuntimeError(f"request {request.request_id!r} is already admitted")
        created = self.manager.create_request(request.request_id, lifetime_tokens=request.max_cache_tokens)
        if created is None:
            return False
        self._reservations[request.request_id] = BlockReservation(
            request.request_id, request.max_cache_tokens, tuple(created.promised))
        return True

    def release_finished(self, request_ids: tuple[str, ...]) -> dict[str, dict[int, list[int]]]:
        return self.release_admitted(request_ids)

    def release_admitted(self, request_ids: tuple[str, ...]) -> dict[str, dict[int, list[int]]]:
        """Give back the pages and promises of these requests (finished, or admitted in a step
        that failed).  Returns the freed page ids per request and cache group."""
        if len(set(request_ids)) != len(request_ids):
            raise ValueError("request ids must not repeat")
        missing = [rid for rid in request_ids if rid not in self._reservations]
        if missing:
            raise KeyError(f"requests without a page reservation: {missing}")
        released = {}
        for request_id in request_ids:
            released[request_id] = self.manager.release(request_id)
            del self._reservations[request_id]
        return released
