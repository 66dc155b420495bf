"""The Python entry point, in the manner of hari495/dryft's ``Engine`` (``engine/engine.py:28-30,138-140``):

    eng = Engine(model_path)
    for step in eng.generate(input_ids, max_new_tokens):   # one list of token ids per step
        ...

``Engine(model_path)`` reads ``config.json``, picks the architecture from its ``architectures``, loads
``model.safetensors`` by tensor name, builds the cache and compiles the kernels the model's sizes
need.  There is no CPU path: a CUDA device and a working nvcc build are required, and their absence
is an error, not a fallback.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Iterator, List, Mapping, Optional, Sequence, Union

import torch

from ..cache.store import SequenceCache
from ..config import config_from_dict, load_config
from ..parts.base import Runtime
from ..sampling.sampler import SamplingParams, choose
from ..weights import Checkpoint, CheckpointSource, RandomSource, expected_tensors
from .loop import ENDED, plan_batches, run_batch, run_requests
from .model import DecoderModel
from .step import Stepper

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, torch.float32: torch.float32,
}


@dataclass
class EngineOptions:
    """Capacities and switches (the reference's ``Settings``, ``engine/dryft_qwen3/config.py:161-193``,
    without buckets: ``b_max=32``, ``l_max=8192`` are its defaults too)."""

    dtype: Union[str, torch.dtype] = "bfloat16"
    max_batch: int = 32
    max_seq_len: Optional[int] = None      # default: min(max_position_embeddings, 8192)
    max_tokens: Optional[int] = None       # cache size in tokens; default max_batch * max_seq_len
    page_size: int = 64
    cuda_graphs: bool = True
    device: str = "cuda:0"
    small_m_max: int = 16                   # rows up to which decode products stream weights through registers (mma.sync)
    stream_m_max: int = 0                  # rows up to which they stream them by TMA into tcgen05.mma above that (0: cuBLAS,
                                           # which is faster today: profiles/gemm_stream_microbench.md)
    fuse_decode: bool = True               # fold norms, adds and SiLU*mul into the decode products
    pdl: bool = True                       # programmatic dependent launch between the decode products
    # fused decode: the next norm's weight is applied by the product before it and the norm's factor by the product
    # behind it.  3 % faster at batch 1 to 8, but the activations are then rounded once where the reference rounds twice
    # (engine/dryft_qwen3/model.py:28-32): as close to 32-bit as the default, 1.3 times further from a plain bfloat16
    # evaluation.  Off by default: the default path keeps the reference's rounding points.
    norm_ahead: bool = False
    tcgen05: bool = True                   # prefill attention on tcgen05 / TMEM / TMA where the head size allows
    # Prompts longer than this go through the step function in chunks of this many tokens per sequence (the same
    # step again, from the cache the chunk before left): bounds the step's activations ([tokens, q + 2 kv], the
    # attention output) whatever the prompt length.  None: whole prompts in one step.
    prefill_chunk_tokens: Optional[int] = None


def _require_cuda(device: str) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("dryft_b200 needs a CUDA device (built for NVIDIA B200, sm_100a); none is available "
                           "and there is no CPU path")
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"dryft_b200 runs on CUDA devices only, got {device!r}")
    return dev


class Engine:
    def __init__(self, model_path: str, options: Optional[EngineOptions] = None, **kw: Any):
        opts = options or EngineOptions(**kw)
        config = load_config(model_path)
        ckpt = Checkpoint(model_path)
        spec = config.model_spec()
        ckpt.check(expected_tensors(spec))
        dev = _require_cuda(opts.device)
        dtype = _DTYPES[opts.dtype]
        self._build(config, spec, CheckpointSource(ckpt, dtype, dev), opts, dev, dtype)

    @classmethod
    def from_config(cls, config: Union[Mapping[str, Any], Any], seed: int = 0, std: float = 0.02,
                    options: Optional[EngineOptions] = None, draw_on: str = "device", **kw: Any) -> "Engine":
        """Random weights without a model folder.  ``draw_on="device"`` draws them with the GPU's generator
        (seconds for billions of values: benchmarks of large shapes); ``draw_on="cpu"`` draws them with the CPU's
        generator, tensor by tensor -- exactly the tensors ``write_random_model(config, seed, ...)`` stores, so a
        seed then names one model whether it is written to a folder or built here.  The two generators give
        different values for the same seed."""
        if draw_on not in ("device", "cpu"):
            raise ValueError(f"draw_on must be 'device' or 'cpu', got {draw_on!r}")
        self = cls.__new__(cls)
        opts = options or EngineOptions(**kw)
        cfg = config_from_dict(config) if isinstance(config, Mapping) else config
        spec = cfg.model_spec()
        dev = _require_cuda(opts.device)
        dtype = _DTYPES[opts.dtype]
        exp = expected_tensors(spec)
        skip = [n for n, info in exp.items() if info.optional]
        source = RandomSource(exp, seed, dtype, dev, std=std, skip=skip,
                              draw_device=torch.device("cpu") if draw_on == "cpu" else dev)
        self._build(cfg, spec, source, opts, dev, dtype)
        return self

    def _build(self, config, spec, source, opts: EngineOptions, dev: torch.device, dtype: torch.dtype) -> None:
        torch.backends.cuda.matmul.allow_tf32 = False  # engine/engine.py:32-33
        torch.backends.cudnn.allow_tf32 = False
        if opts.prefill_chunk_tokens is not None and opts.prefill_chunk_tokens <= 0:
            raise ValueError(f"prefill_chunk_tokens must be positive, got {opts.prefill_chunk_tokens}")
        self.config = config
        self.spec = spec
        self.options = opts
        self.device = dev
        self.dtype = dtype
        props = torch.cuda.get_device_properties(dev)
        self.rt = Runtime(dtype=dtype, device=dev, page_size=opts.page_size, sm_count=props.multi_processor_count,
                          small_m_max=opts.small_m_max, stream_m_max=opts.stream_m_max, fuse_decode=opts.fuse_decode, pdl=opts.pdl, tcgen05=opts.tcgen05, norm_ahead=opts.norm_ahead)
        with torch.cuda.device(dev), torch.no_grad():
            self.model = DecoderModel(spec, source, self.rt)
            self.max_seq_len = opts.max_seq_len or min(spec.max_positions, 8192)
            self.max_batch = opts.max_batch
            self.max_tokens = opts.max_tokens or self.max_batch * _round_up(self.max_seq_len, opts.page_size)
            needs, borrow = self.model.cache_needs()
            self.cache = SequenceCache(needs, borrow, max_tokens=self.max_tokens, max_slots=self.max_batch,
                                       max_seq_len=self.max_seq_len, page_size=opts.page_size, dtype=dtype, device=dev)
            self.stepper = Stepper(self.model, self.cache, self.rt, cuda_graphs=opts.cuda_graphs)
        self._backend = _DeviceBackend(self)

    # ------------------------------------------------------------------ generation
    def generate(self, input_ids: Sequence[Sequence[int]], max_new_tokens: int, *, temperature: float = 0.0,
                 top_k: int = 0, seed: int = 0, stop_token_ids: Sequence[int] = ()) -> Iterator[List[int]]:
        """Yield one list of token ids per step, one id per sequence (``-1`` once a sequence has ended at
        a stop token).  With no stop tokens: exactly ``max_new_tokens`` lists (``engine/engine.py:138-140``).
        The sequences start together as one batch; use ``generate_many`` for more requests than fit."""
        params = SamplingParams(temperature, top_k, seed)
        B = len(input_ids)
        if B > self.max_batch:
            raise ValueError(f"{B} sequences in one batch; the engine was built for max_batch={self.max_batch} "
                             "(generate_many runs batches one after another)")
        final = [len(p) + max_new_tokens for p in input_ids]
        if B and max_new_tokens > 0 and not self.cache.can_hold(final):
            raise ValueError(f"batch does not fit the cache: final lengths {final}, {self.cache.free_tokens()} tokens free, "
                             f"max_seq_len {self.max_seq_len}")
        with torch.cuda.device(self.device), torch.inference_mode():
            yield from run_batch(self._backend, input_ids, max_new_tokens, params, stop_token_ids)

    def generate_many(self, input_ids: Sequence[Sequence[int]], max_new_tokens: int, *, temperature: float = 0.0,
                      top_k: int = 0, seed: int = 0, stop_token_ids: Sequence[int] = ()) -> List[List[int]]:
        """Any number of requests, run as batches one after another; returns the new tokens of each."""
        params = SamplingParams(temperature, top_k, seed)
        if max_new_tokens <= 0 or not input_ids:
            return [[] for _ in input_ids]
        for p in input_ids:
            if len(p) == 0:
                raise ValueError("empty prompt")
        batches = plan_batches([len(p) + max_new_tokens for p in input_ids], self.max_batch, self.max_tokens,
                               self.options.page_size, self.max_seq_len)
        with torch.cuda.device(self.device), torch.inference_mode():
            return run_requests(self._backend, input_ids, max_new_tokens, params, stop_token_ids, batches)


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class _DeviceBackend:
    """The loop's backend on the GPU: prompts through ``Stepper.step``, decode steps through the
    captured decode graph fed from the per-sequence state, token choice by the sampling kernels."""

    def __init__(self, engine: Engine):
        self.e = engine
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._seq_key = None
        self._seq_dev = None
        self._ring = None      # pinned buffers for the chosen tokens of the steps in flight
        self._ring_at = 0

    def open(self, n: int) -> List[int]:
        return self.e.cache.open_sequences(n)

    def close(self, handles: Sequence[int]) -> None:
        self.e.cache.close_sequences(handles)
        from ..ops import kernels as K

        K.check_error_flags()  # a kernel that gave up a bounded wait makes the batch's results invalid

    def _ints(self, vals: Sequence[int]) -> torch.Tensor:
        return torch.tensor(list(vals), dtype=torch.int32).to(self.e.device, non_blocking=True)

    def _prompt_logits(self, handles, prompts) -> torch.Tensor:
        """Logits at each prompt's last token: one step, or the same step chunk after chunk."""
        e = self.e
        chunk = e.options.prefill_chunk_tokens
        longest = max(len(p) for p in prompts)
        if not chunk or longest <= chunk:
            return e.stepper.step(handles, prompts, [[len(p) - 1] for p in prompts])
        rows: List[Optional[torch.Tensor]] = [None] * len(prompts)
        for c0 in range(0, longest, chunk):
            live = [b for b, p in enumerate(prompts) if len(p) > c0]      # shorter prompts are done already
            pieces = [prompts[b][c0:c0 + chunk] for b in live]
            ends = [len(prompts[b]) <= c0 + chunk for b in live]          # this piece holds the prompt's last token
            out = e.stepper.step([handles[b] for b in live], pieces, [[len(pc) - 1] if end else [] for pc, end in zip(pieces, ends)])
            at = 0
            for b, end in zip(live, ends):
                if end:
                    rows[b] = out[at:at + 1]
                    at += 1
        return torch.cat(rows)

    def prefill(self, handles, prompts, seq_ids, params: SamplingParams) -> List[int]:
        e = self.e
        logits = self._prompt_logits(handles, prompts)
        chosen = choose(logits, params, row_seq=self._ints(seq_ids), step=0, row_slot=self._ints(handles),
                        last_token=e.cache.last_token)
        self.h2d_bytes += 4 * (sum(len(p) for p in prompts) + 4 * len(prompts))
        self.d2h_bytes += 4 * len(prompts)
        return chosen.tolist()

    def decode(self, handles, seq_ids, step: int, params: SamplingParams) -> List[int]:
        return self.decode_result(self.decode_launch(handles, seq_ids, step, params))

    def decode_launch(self, handles, seq_ids, step: int, params: SamplingParams):
        """Start a decode step: the graph, the token choice and the copy of the chosen tokens into pinned
        memory are queued; nothing waits.  The ticket is redeemed by ``decode_result``."""
        e = self.e
        n = len(handles)
        logits = e.stepper.decode_from_state(handles)
        bucket = logits.shape[0]
        row_seq = None
        if not params.greedy:
            key = tuple(seq_ids) + (bucket,)
            if self._seq_key != key:  # changes only when a sequence leaves the batch
                self._seq_key, self._seq_dev = key, self._ints(list(seq_ids) + [0] * (bucket - n))
                self.h2d_bytes += 4 * bucket
            row_seq = self._seq_dev
        chosen = choose(logits, params, row_seq=row_seq, step=step, row_slot=e.stepper.last_decode_slots,
                        last_token=e.cache.last_token)
        self.h2d_bytes += 4 * bucket  # the step's slot list, staged in pinned memory
        self.d2h_bytes += 4 * n
        if self._ring is None or self._ring[0].numel() < bucket:
            self._ring = [torch.empty(max(bucket, 64), dtype=torch.int32).pin_memory() for _ in range(4)]
            self._ring_at = 0
        host = self._ring[self._ring_at]
        self._ring_at = (self._ring_at + 1) % len(self._ring)
        host[:n].copy_(chosen[:n], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return host, n, done

    def decode_result(self, ticket) -> List[int]:
        host, n, done = ticket
        done.synchronize()
        return host[:n].tolist()
