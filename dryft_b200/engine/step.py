"""The one step function.

A step is a batch of sequences that either all start (their prompts, of unequal lengths, packed
back to back) or all go on by one token.  It runs only the tokens it is given, as one batch, from
the cache that earlier steps left, and returns 32-bit logits at the wanted places.  Sequence ``b``
appends ``q_len[b]`` tokens at positions ``len .. len + q_len - 1`` of its slot, and the token at
position ``p`` sees keys ``0..p`` — the reference's chain semantics
(``engine/dryft_qwen3/model.py:307-318``; ``kernels/attn_decode.py:46-63``), which make prefill, chunked
prefill and decode the same operation.  The reference has two entry points instead (equal-length
``prefill`` groups and ``decode_step``, ``model.py:123,191``) and runs ragged batches as several
prefills (``engine/engine.py:172-186``).

Padding: a decode batch may be padded to a captured size with sequences whose slot is -1; every
kernel skips them, so padding changes no result.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.store import SequenceCache
from ..ops import kernels as K
from ..parts.base import Runtime, StepContext
from .model import DecoderModel


class Stepper:
    def __init__(self, model: DecoderModel, cache: SequenceCache, rt: Runtime, cuda_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.rt = rt
        self.cuda_graphs = cuda_graphs
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}
        self._pinned: Optional[torch.Tensor] = None
        self._upload_event: Optional[torch.cuda.Event] = None
        # query tokens per prefill tile: the smallest any mixer asks for (64 unless every mixer takes more)
        self.prefill_tile = min([getattr(b.mixer, "prefill_tile", 64) for b in model.blocks] or [64])
        self.last_decode_slots: Optional[torch.Tensor] = None
        self._prompt_graphs: Dict[tuple, "_PromptGraph"] = {}   # (tokens, sequences, wanted rows, tiles) -> captured step
        self._prompt_shapes_seen: set = set()

    # ------------------------------------------------------------------ host -> device metadata
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Sequence[Sequence[int]]) -> Optional[torch.Tensor]:
        """``slots[b]`` appends ``tokens[b]``; logits are returned for ``want[b]`` (indices into
        ``tokens[b]``), in the order of the sequences and of ``want``: ``[n_wanted, vocab]`` float32
        on the device, or None when nothing is wanted."""
        B = len(slots)
        if B == 0:
            return None
        if len(tokens) != B or len(want) != B:
            raise ValueError("step: slots, tokens and want must have one entry per sequence")
        vocab = self.model.vocab_size
        q_lens = [len(t) for t in tokens]
        if any(q == 0 for q in q_lens):
            raise ValueError("step: every sequence of a step brings at least one token")
        if len(set(slots)) != B:
            raise ValueError("step: a slot occurs twice in one step")
        # the step's integers as arrays: a prompt of thousands of tokens is checked and packed at once
        parts = [np.asarray(t.cpu() if isinstance(t, torch.Tensor) else t) for t in tokens]
        if any(a.dtype.kind not in "iu" for a in parts):
            parts = [np.asarray([int(v) for v in t], dtype=np.int64) for t in tokens]
        flat = np.concatenate(parts).astype(np.int64, copy=False)
        if flat.size and (int(flat.min()) < 0 or int(flat.max()) >= vocab):
            bad = int(flat[(flat < 0) | (flat >= vocab)][0])
            raise ValueError(f"step: token id {bad} is outside the vocabulary [0, {vocab})")
        cu = [0]
        for q in q_lens:
            cu.append(cu[-1] + q)
        rows: List[int] = []
        for b, w in enumerate(want):
            for i in w:
                if not 0 <= int(i) < q_lens[b]:
                    raise ValueError(f"step: wanted place {i} is outside the {q_lens[b]} tokens of sequence {b}")
                rows.append(cu[b] + int(i))
        decode = all(q == 1 for q in q_lens)
        starts = [self.cache.len_host[s] for s in slots]

        for s, q in zip(slots, q_lens):
            self.cache.reserve(s, q)
        self.cache.flush()

        N = int(flat.size)
        tiles0: List[int] = []
        tilesn: List[int] = []
        if not decode:
            order = []
            for b, q in enumerate(q_lens):
                for q0 in range(0, q, self.prefill_tile):
                    order.append((starts[b] + q0, cu[b] + q0, min(self.prefill_tile, q - q0)))
            order.sort(key=lambda t: -t[0])  # tiles with the most keys first
            tiles0 = [t[1] for t in order]
            tilesn = [t[2] for t in order]
        T = len(tiles0)
        W = len(rows)
        packed = np.concatenate((flat, np.asarray(cu + list(slots) + rows + tiles0 + tilesn, dtype=np.int64))).astype(np.int32)
        max_kv = max(st + q for st, q in zip(starts, q_lens))
        logits = None
        shape = (N, B, W, T)
        if self.cuda_graphs and not decode and N >= self.PROMPT_GRAPH_MIN_TOKENS:
            # A prompt step's launches depend on these four counts only (every length, position, slot and tile is
            # data the kernels read on the device), so a step of a shape seen before is replayed from a captured
            # graph: the host's lead before the first launch and the gaps between some hundred launches go away.
            g = self._prompt_graphs.get(shape)
            if g is not None:
                self._prompt_graphs[shape] = self._prompt_graphs.pop(shape)     # most recently used last
                self._upload(packed, into=g.ints)
                logits = g.replay()
            elif shape in self._prompt_shapes_seen:                             # second time: worth a capture
                g = _PromptGraph(self, shape, int(packed.size))
                self._upload(packed, into=g.ints)
                g.capture()
                logits = g.replay()
                self._prompt_graphs[shape] = g
                while len(self._prompt_graphs) > self.PROMPT_GRAPHS_KEPT:       # each holds its activations: keep a few
                    self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
            else:
                self._prompt_shapes_seen.add(shape)
                g = None
        else:
            g = None
        if g is None:
            dev = self._upload(packed)
            meta = torch.empty(2 * N, dtype=torch.int32, device=self.rt.device)
            logits = self._run(dev, meta, shape, decode, max_kv)
        for s, q in zip(slots, q_lens):
            self.cache.advanced(s, q)
        return logits

    PROMPT_GRAPH_MIN_TOKENS = 256   # below this a step is too short for its launches to matter
    PROMPT_GRAPHS_KEPT = 4

    def _run(self, dev: torch.Tensor, meta: torch.Tensor, shape, decode: bool, max_kv: int) -> Optional[torch.Tensor]:
        """The device side of a step: ``dev`` holds the step's integers as ``step`` packs them."""
        N, B, W, T = shape
        o = 0
        d_tokens = dev[o:o + N]; o += N
        d_cu = dev[o:o + B + 1]; o += B + 1
        d_slot = dev[o:o + B]; o += B
        d_rows = dev[o:o + W]; o += W
        d_t0 = dev[o:o + T]; o += T
        d_tn = dev[o:o + T]; o += T
        tok_slot, tok_pos = meta[:N], meta[N:]
        K.step_meta(d_cu, d_slot, self.cache.seq_len, tok_slot, tok_pos, N, B)
        ctx = StepContext(n_tokens=N, n_seqs=B, tokens=d_tokens, cu_q=d_cu, seq_slot=d_slot, tok_slot=tok_slot,
                          tok_pos=tok_pos, decode=decode, max_kv=max_kv,
                          tile_tok0=d_t0 if T else None, tile_rows=d_tn if T else None, n_tiles=T, tile_size=self.prefill_tile)
        logits = self.model.forward(ctx, self.cache, d_rows if W else None, W)
        K.step_advance(d_cu, d_slot, self.cache.seq_len, B)
        return logits

    def _upload(self, ints: np.ndarray, into: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One host->device copy of the step's integers (an int32 array) through pinned memory, into a fresh device
        tensor or into ``into`` (a captured graph's own buffer)."""
        n = int(ints.size)
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
        # the previous step's copy out of this buffer must have finished before it is rewritten
        if self._upload_event is not None:
            self._upload_event.synchronize()
        buf = self._pinned[:n]
        buf.numpy()[:] = ints
        dev = torch.empty(n, dtype=torch.int32, device=self.rt.device) if into is None else into[:n]
        dev.copy_(buf, non_blocking=True)
        self._upload_event = torch.cuda.Event()
        self._upload_event.record()
        return dev

    # ------------------------------------------------------------------ decode from the device state
    def decode_from_state(self, slots: Sequence[int]) -> torch.Tensor:
        """One decode step whose input tokens are the sequences' last chosen tokens, kept on the
        device (``SequenceCache.last_token``).  Returns logits ``[bucket, vocab]``; rows beyond
        ``len(slots)`` belong to padding.  Replays a captured CUDA graph of the step when enabled
        (one graph per batch size serves every position, because lengths are read on the device —
        ``engine/dryft_qwen3/cache.py:8-10``; ``graphs.py:108-135``)."""
        B = len(slots)
        for s in slots:
            self.cache.reserve(s, 1)
        self.cache.flush()
        bucket = _bucket(B)
        # one graph per (batch size, context bucket): the context bucket only decides how the decode
        # attention splits its keys across blocks (the reference buckets lengths too, config.py:169-170)
        kv_bucket = _kv_bucket(max(self.cache.len_host[s] for s in slots) + 1)
        g = self._graphs.get((bucket, kv_bucket))
        if g is None:
            g = _DecodeGraph(self, bucket, kv_bucket)
            self._graphs[(bucket, kv_bucket)] = g
        logits = g.run(slots)
        for s in slots:
            self.cache.advanced(s, 1)
        self.last_decode_slots = g.seq_slot  # int32 [bucket] on the device, -1 for padding rows
        return logits


class _PromptGraph:
    """A captured prompt step of one shape: its own copy of the step's integers, its token metadata and the graph.
    The reference captures decode steps only (``engine/dryft_qwen3/graphs.py:25-59``); its prompts run eagerly."""

    def __init__(self, stepper: Stepper, shape, n_ints: int):
        self.st = stepper
        self.shape = shape
        dev = stepper.rt.device
        self.ints = torch.zeros(n_ints, dtype=torch.int32, device=dev)
        self.meta = torch.empty(2 * shape[0], dtype=torch.int32, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.n_kernels = 0

    def capture(self) -> None:
        """The eager run of this shape that came before was the warm-up (library workspaces, kernel attributes)."""
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        before = K.launch_count
        with torch.cuda.graph(self.graph):
            self.logits = self.st._run(self.ints, self.meta, self.shape, False, 0)
        self.n_kernels = K.launch_count - before

    def replay(self) -> Optional[torch.Tensor]:
        self.graph.replay()
        K.launch_count += self.n_kernels
        # the graph writes its logits in place: hand out a copy, the next replay must not change what a caller keeps
        return None if self.logits is None else self.logits.clone()


def _bucket(b: int) -> int:
    """Decode batch sizes are padded to 1, 2, 4, 8, then multiples of 8."""
    if b <= 8:
        n = 1
        while n < b:
            n *= 2
        return n
    return (b + 7) // 8 * 8


def _kv_bucket(n: int) -> int:
    """Context lengths are bucketed to 1024, 2048, 4096, ..."""
    b = 1024
    while b < n:
        b *= 2
    return b


class _DecodeGraph:
    """Static buffers and (optionally) a captured graph of one decode step at a fixed batch size and
    context bucket."""

    def __init__(self, stepper: Stepper, bucket: int, kv_bucket: int):
        self.st = stepper
        self.bucket = bucket
        self.kv_bucket = kv_bucket
        dev = stepper.rt.device
        # pinned staging for the per-step slot list: a ring, so the host may run several steps ahead
        self.ring = [torch.full((bucket,), -1, dtype=torch.int32).pin_memory() for _ in range(8)]
        self.ring_events: list = [None] * 8
        self.ring_at = 0
        self.seq_slot = torch.full((bucket,), -1, dtype=torch.int32, device=dev)
        self.cu_q = torch.arange(bucket + 1, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(bucket, dtype=torch.int32, device=dev)
        self.tok_slot = torch.zeros(bucket, dtype=torch.int32, device=dev)
        self.tok_pos = torch.zeros(bucket, dtype=torch.int32, device=dev)
        self.rows = torch.arange(bucket, dtype=torch.int32, device=dev)
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.h2d_bytes = 4 * bucket
        self.n_kernels = 0      # launches of this library's kernels in one step

    def _body(self) -> torch.Tensor:
        st = self.st
        K.tokens_from_state(self.seq_slot, st.cache.last_token, self.tokens, self.bucket)
        K.step_meta(self.cu_q, self.seq_slot, st.cache.seq_len, self.tok_slot, self.tok_pos, self.bucket, self.bucket)
        ctx = StepContext(n_tokens=self.bucket, n_seqs=self.bucket, tokens=self.tokens, cu_q=self.cu_q,
                          seq_slot=self.seq_slot, tok_slot=self.tok_slot, tok_pos=self.tok_pos, decode=True,
                          max_kv=self.kv_bucket)
        logits = st.model.forward(ctx, st.cache, self.rows, self.bucket, all_rows=True)
        K.step_advance(self.cu_q, self.seq_slot, st.cache.seq_len, self.bucket)
        return logits

    def run(self, slots: Sequence[int]) -> torch.Tensor:
        n = len(slots)
        i = self.ring_at
        self.ring_at = (i + 1) % len(self.ring)
        if self.ring_events[i] is not None:
            self.ring_events[i].synchronize()  # the copy that last used this staging buffer has finished
        host = self.ring[i]
        host[:n] = torch.tensor(list(slots), dtype=torch.int32)
        host[n:] = -1
        self.seq_slot.copy_(host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.ring_events[i] = ev
        if not self.st.cuda_graphs:
            return self._body()
        if self.graph is None:
            # Capture.  Warm-up runs would advance the sequences, so they run on padding only.
            torch.cuda.synchronize()
            self.seq_slot.fill_(-1)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            before = K.launch_count
            with torch.cuda.graph(self.graph):
                self.logits = self._body()
            self.n_kernels = K.launch_count - before
            self.seq_slot.copy_(host, non_blocking=True)
        self.graph.replay()
        K.launch_count += self.n_kernels
        return self.logits
