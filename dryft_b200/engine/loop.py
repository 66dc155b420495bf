"""The generation loop: what runs in which step, when a sequence ends, what is yielded.

Everything here is host logic over an abstract backend, so it is tested on the CPU with a scripted
backend.  The shape of the API follows ``engine/engine.py:138-166,192-234`` of hari495/dryft:
``generate(input_ids, max_new_tokens)`` yields one list of token ids per step, one id per sequence,
the first from the prompts' step.  Differences, on purpose: prompts of unequal lengths run in ONE
step (the reference groups them by length, ``engine.py:172-186``); a sequence may stop early at a
stop token (the reference never stops, ``engine.py:139-140``) — it is then left out of later steps
and its entry in later yields is -1; the loop ends when every sequence has ended.  Without stop tokens
the host need not see step t's tokens before step t+1 runs (the tokens stay on the device), so a backend
that offers ``decode_launch`` / ``decode_result`` keeps one step in flight: step t+1 is launched before
step t's tokens are read, as the reference does with its pinned ring (``engine.py:215-229``).
"""

from __future__ import annotations

from typing import Iterator, List, Protocol, Sequence

from ..sampling.sampler import SamplingParams

ENDED = -1


class Backend(Protocol):
    """What the loop drives.  ``handles`` are opaque per-sequence tickets (cache slots)."""

    def open(self, n: int) -> List[int]: ...
    def prefill(self, handles: Sequence[int], prompts: Sequence[Sequence[int]], seq_ids: Sequence[int],
                params: SamplingParams) -> List[int]: ...
    def decode(self, handles: Sequence[int], seq_ids: Sequence[int], step: int, params: SamplingParams) -> List[int]: ...
    def close(self, handles: Sequence[int]) -> None: ...
    # optional pair: ``decode_launch(handles, seq_ids, step, params) -> ticket`` starts a decode step without
    # waiting for it, ``decode_result(ticket) -> List[int]`` waits for that step and returns its tokens


def check_request(input_ids: Sequence[Sequence[int]], max_new_tokens: int) -> None:
    for i, p in enumerate(input_ids):
        if len(p) == 0:
            raise ValueError("empty prompt")  # engine/engine.py:176-177
    if max_new_tokens < 0:
        raise ValueError(f"max_new_tokens must be >= 0, got {max_new_tokens}")


def run_batch(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens: int, params: SamplingParams,
              stop_token_ids: Sequence[int] = (), seq_ids: Sequence[int] = ()) -> Iterator[List[int]]:
    """One batch of sequences that start together.  Yields a list per step: the chosen token of each
    sequence, or ``ENDED`` for a sequence that ended at an earlier step.  A stop token is yielded,
    then its sequence ends.  Slots are given back when the batch ends (also on error or when the
    consumer stops early)."""
    B = len(prompts)
    if B == 0 or max_new_tokens <= 0:  # engine/engine.py:142-143
        return
    check_request(prompts, max_new_tokens)
    seq_ids = list(seq_ids) if seq_ids else list(range(B))
    stops = set(int(t) for t in stop_token_ids)
    handles = backend.open(B)
    try:
        alive = list(range(B))
        toks = backend.prefill(handles, prompts, seq_ids, params)
        step = 0
        if not stops and hasattr(backend, "decode_launch") and hasattr(backend, "decode_result"):
            # nobody can end early: every step runs all sequences, and one step is kept in flight
            yield [int(t) for t in toks]          # the first tokens go out before any decode step is launched
            if max_new_tokens == 1:
                return
            ticket = backend.decode_launch(handles, seq_ids, 1, params)
            for step in range(1, max_new_tokens):
                ahead = backend.decode_launch(handles, seq_ids, step + 1, params) if step + 1 < max_new_tokens else None
                yield [int(t) for t in backend.decode_result(ticket)]
                ticket = ahead
            return
        while True:
            out = [ENDED] * B
            for b, t in zip(alive, toks):
                out[b] = int(t)
            yield out
            step += 1
            alive = [b for b in alive if out[b] not in stops]
            if step >= max_new_tokens or not alive:
                return
            toks = backend.decode([handles[b] for b in alive], [seq_ids[b] for b in alive], step, params)
    finally:
        backend.close(handles)


def plan_batches(final_lengths: Sequence[int], max_batch: int, max_tokens: int, page_size: int, max_seq_len: int) -> List[List[int]]:
    """Cut requests (in order) into batches that fit the cache: at most ``max_batch`` sequences and
    at most ``max_tokens`` tokens, each sequence's final length rounded up to whole pages."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(final_lengths):
        if n > max_seq_len:
            raise ValueError(f"request {i} needs {n} tokens; the engine was built for sequences of at most {max_seq_len}")
        need = (n + page_size - 1) // page_size * page_size
        if need > max_tokens:
            raise ValueError(f"request {i} needs {need} cache tokens; the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def run_requests(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens: int, params: SamplingParams,
                 stop_token_ids: Sequence[int], batches: Sequence[Sequence[int]]) -> List[List[int]]:
    """As many batches one after another as there are requests; returns each request's new tokens
    (a stop token included, nothing after it).  Request ``i`` samples as sequence ``i`` whatever batch
    it lands in."""
    results: List[List[int]] = [[] for _ in prompts]
    for batch in batches:
        for step_tokens in run_batch(backend, [prompts[i] for i in batch], max_new_tokens, params, stop_token_ids,
                                     seq_ids=list(batch)):
            for i, t in zip(batch, step_tokens):
                if t != ENDED:
                    results[i].append(t)
    return results
