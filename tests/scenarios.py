"""Ways of cutting the same requests into steps.  Every function returns a list of steps; a step
is ``{"entries": [(request_id, start, end), ...], "end": [request_id, ...]}`` meaning: feed tokens
start..end-1 of that request in this step.  All logits are always wanted, so that every position
of every request can be compared with the plain implementation run on the request alone, whole."""

from __future__ import annotations

import random


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, in one step."""
    return [{"entries": [(rid, 0, len(tokens))], "end": [rid]} for rid, tokens in requests.items()]


def tail_one_by_one(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(len(tokens) - tail, 0)
        if head:
            steps.append({"entries": [(rid, 0, head)], "end": []})
        for position in range(head, len(tokens)):
            steps.append({"entries": [(rid, position, position + 1)],
                          "end": [rid] if position == len(tokens) - 1 else []})
    return steps


def changing_portions(requests: dict[str, list[int]], sizes=(7, 2, 16, 3, 33, 2, 17, 64, 5, 31)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, tokens in requests.items():
        start, turn = 0, 0
        while start < len(tokens):
            end = min(len(tokens), start + sizes[turn % len(sizes)])
            steps.append({"entries": [(rid, start, end)], "end": [rid] if end == len(tokens) else []})
            start, turn = end, turn + 1
    return steps


def mixed(requests: dict[str, list[int]], seed: int, max_live: int = 4, decode_tail: int = 12) -> list[dict]:
    """Up to ``max_live`` requests at a time; each step gives some of them a portion of their
    prompt, others a single token (their last ``decode_tail`` tokens come one by one), and leaves
    some out.  Requests start as others end, so that freed pages are used again."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            live[waiting.pop(0)] = 0
        entries, ended = [], []
        for rid in list(live):
            total = len(requests[rid])
            done = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step
            if total - done <= decode_tail:
                count = 1
            else:
                count = min(rng.choice((2, 3, 5, 8, 13, 16, 17, 31, 40)), total - done - decode_tail)
            entries.append((rid, done, done + count))
            live[rid] = done + count
            if live[rid] == total:
                ended.append(rid)
        for rid in ended:
            del live[rid]
        if entries:
            rng.shuffle(entries)
            steps.append({"entries": entries, "end": ended})
    return steps


def pool_tokens(requests: dict[str, list[int]], steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for rid, _, end in step["entries"]:
            held[rid] = end
        peak = max(peak, sum(-(-count // round_to) * round_to for count in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak
