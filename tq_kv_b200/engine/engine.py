"""The engine: a model, its cache and the one step function.

`Engine.step(rows)` runs the tokens each row brings — whole prompts of unequal
length in one step, or one token per sequence — as one packed batch from the
cache and returns float32 logits at the wanted places.  Generation
(`Engine.generate`, generate.py) and trace replay (replay.py) are loops above
this one function.

Reference: src/engine.rs:231-319 (load), :365-370 and :395-400 (the two
forward calls per request that `step` generalises), :322-324 (clear_cache).
There is no CPU path: the device must be a CUDA device.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels
from ..cache import PAGE_TOKENS, CacheError, SequenceCache, StepError
from ..config import read_config_json, spec_from_config_dict
from ..parts import Runtime
from ..weights import load_tensors, random_tensors
from ..weights.random_init import storage_dtype
from .batch import FlatRows, StepRow, build_step_batch
from .decode_graph import DecodeGraph, PromptGraph, forward_step
from .readback import SampledIds
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class Engine:
    def __init__(self, model: DecoderModel, config, config_dict: dict, runtime: Runtime, cache: SequenceCache):
        self.model = model
        self.config = config
        self.config_dict = config_dict
        self.runtime = runtime
        self.cache = cache
        self.spec = model.spec
        self.vocab_size = model.spec.vocab_size
        self.steps_run = 0
        self.use_graphs = model.graph_capturable      # replay captured CUDA graphs for decode steps
        self._decode_graphs: dict[int, "DecodeGraph"] = {}
        # single prompts from position 0 replay graphs too, padded to a few sizes (PromptGraph)
        self.pad_prompts = model.padded_rows_ok and not cache.state
        self._prompt_graphs: dict[tuple, "PromptGraph"] = {}
        self._prompt_pool = None
        self.h2d_bytes = 0            # bytes of step inputs copied to the device so far
        self.sampled = SampledIds(runtime.device)     # where the sampler's ids go; rows may name them as source

    # ---- construction -------------------------------------------------------
    @classmethod
    def _build(cls, config_dict: dict, tensors_for, *, dtype, device, max_tokens: Optional[int],
               max_slots: Optional[int], max_context: Optional[int], window_chunk: int = 64) -> "Engine":
        """`window_chunk`: the most tokens a step may add to a sequence that it
        continues (a portion of a prompt, a prompt beside decoding rows) in a
        layer with a sliding window; such a layer keeps window + window_chunk - 1
        keys per sequence, rounded up to whole pages."""
        if window_chunk < 1:
            raise ValueError("window_chunk must be at least 1")
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', not {dtype!r}")
        mode = _DTYPES[dtype]
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("this engine runs on a CUDA device only (there is no CPU path)")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; the engine cannot run")
        arch, cfg, spec = spec_from_config_dict(config_dict)
        model = DecoderModel(spec)
        # cache geometry: context limit, then tokens held together, then slots
        if max_context is None:
            max_context = spec.max_positions if max_tokens is None else min(spec.max_positions,
                                                                            _round_up(max_tokens, PAGE_TOKENS))
        if max_context > spec.max_positions:
            raise ValueError(f"max_context {max_context} exceeds the model's max positions {spec.max_positions}")
        if max_tokens is None:
            max_tokens = (max_slots or 1) * _round_up(max_context, PAGE_TOKENS)
        if max_slots is None:
            max_slots = max(1, -(-max_tokens // PAGE_TOKENS))
        runtime = Runtime(device=dev, act_dtype=mode, max_context=max_context, window_chunk=window_chunk)
        with torch.cuda.device(dev):
            model.bind(tensors_for(model, mode, dev), runtime)
            kv_req, state_req = model.cache_requests()
            cache = SequenceCache(kv_req, state_req, max_tokens=max_tokens, max_slots=max_slots,
                                  max_length=max_context, dtype=mode, device=dev, window_slack=window_chunk - 1)
        return cls(model, cfg, config_dict, runtime, cache)

    @classmethod
    def from_folder(cls, folder: str, *, dtype="bfloat16", device="cuda:0", max_tokens: Optional[int] = None,
                    max_slots: Optional[int] = None, max_context: Optional[int] = None,
                    window_chunk: int = 64) -> "Engine":
        """Loads config.json and the safetensors files of `folder`."""
        config_dict = read_config_json(folder)

        def tensors_for(model: DecoderModel, mode, dev):
            expected = {n: tuple(ws.shape) for n, ws in model.weight_specs().items()}
            return load_tensors(folder, expected, model.ignored_weights(), mode=mode, device=dev)

        return cls._build(config_dict, tensors_for, dtype=dtype, device=device, max_tokens=max_tokens,
                          max_slots=max_slots, max_context=max_context, window_chunk=window_chunk)

    @classmethod
    def from_random(cls, config_dict: dict, seed: int = 0, *, dtype="bfloat16", device="cuda:0",
                    max_tokens: Optional[int] = None, max_slots: Optional[int] = None,
                    max_context: Optional[int] = None, window_chunk: int = 64) -> "Engine":
        """Random weights generated on the device (same rules as the folder
        written by `write_model_folder`, without the trip through a file)."""
        def tensors_for(model: DecoderModel, mode, dev):
            stored = storage_dtype(config_dict.get("torch_dtype", "bfloat16"))
            from ..weights.loader import target_dtype
            out = {}
            for name, t in random_tensors(model.weight_specs().values(), seed, stored, dev):
                out[name] = t.to(target_dtype(t.dtype, mode))
            return out

        return cls._build(config_dict, tensors_for, dtype=dtype, device=device, max_tokens=max_tokens,
                          max_slots=max_slots, max_context=max_context, window_chunk=window_chunk)

    # ---- sequences ----------------------------------------------------------
    def new_sequence(self) -> int:
        """A free slot, length 0."""
        return self.cache.alloc_slot()

    def release(self, slot: int) -> None:
        """Gives a slot and everything it holds back."""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step -----------------------------------------------------------
    def _forward(self, batch):
        """One step of the model on a packed batch: tokens that name a source
        are first taken from the sampler's ids on the device."""
        return forward_step(self.model, self.cache, self.sampled.ids, batch)

    def step(self, rows: Sequence[StepRow], *, keep_logits: bool = True, check: bool = True) -> Optional[torch.Tensor]:
        """Runs one step.  Every row brings >= 1 token; its tokens follow what
        the row's slot already holds.  Returns float32 logits [wanted, vocab]
        on the device, in the order of the rows and of each row's `want`
        (None if nothing is wanted).  With `keep_logits` False the result may
        be a buffer that the next step overwrites; with `check` False the step
        does not wait for the device to read the kernels' status word (the
        caller calls check_status() before using the result).  A step that is refused, or
        that fails, changes nothing: lengths stay and the pages it took go back."""
        rows = list(rows)
        if not rows:
            raise StepError("a step needs at least one row")
        try:
            flat = FlatRows(rows)
        except (OverflowError, TypeError, ValueError) as e:
            raise StepError(f"a row's slot, tokens or wanted places are not 32-bit integers: {e}") from e
        # the checks that need no device, then the pages (all rows or none): the host runtime does both
        book = self.cache.book
        book.begin_step(flat.slots, flat.lens, flat.tokens, flat.want_counts, flat.want, flat.sources,
                        self.vocab_size, self.sampled.rows)
        slots, lens = flat.slots, flat.lens
        self.model.check_step(book.lengths(slots), lens.tolist())
        try:
            book.reserve(slots, lens)
        except CacheError as e:
            raise StepError(str(e)) from e
        try:
            with torch.cuda.device(self.runtime.device):
                if self.use_graphs and int(lens.max()) == 1 and all(r.want == [0] for r in rows):
                    graph = self._decode_graphs.get(len(rows))
                    if graph is None:
                        graph = self._decode_graphs[len(rows)] = DecodeGraph(
                            self.model, self.cache, self.sampled.ids, self.runtime, len(rows))
                    logits = graph.run(rows, keep_logits)
                    self.h2d_bytes += graph.batch.packed_bytes
                    kernels.mark_tc_launched()      # read with the sampled ids, or by check_status()
                elif self._prompt_graph_takes(rows, lens):
                    key = (len(rows), -(-int(lens.sum()) // PromptGraph.PAD) * PromptGraph.PAD)
                    graph = self._prompt_graphs.get(key)
                    if graph is None:
                        if self._prompt_pool is None:
                            self._prompt_pool = torch.cuda.graph_pool_handle()     # one pool: they never run together
                        graph = self._prompt_graphs[key] = PromptGraph(
                            self.model, self.cache, self.sampled.ids, self.runtime, key[0], key[1], self._prompt_pool)
                    logits = graph.run(rows)
                    self.h2d_bytes += graph.batch.packed_bytes
                    kernels.mark_tc_launched()
                    if check:
                        kernels.check_tc_status()
                else:
                    batch = build_step_batch(rows, self.cache, self.runtime.device, flat)
                    logits = self._forward(batch)
                    self.h2d_bytes += batch.packed_bytes
                    if check:
                        kernels.check_tc_status()   # a product that gave up on a wait must not pass silently
        except BaseException:
            self.cache.trim(slots)              # the pages taken for this step go back; lengths were not touched
            raise
        self.cache.commit(slots, lens)
        self.steps_run += 1
        return logits

    def _prompt_graph_takes(self, rows, lens) -> bool:
        """Whether the step is whole prompts that may run as a padded, replayed graph (PromptGraph)."""
        if not (self.use_graphs and self.pad_prompts and len(rows) <= PromptGraph.MAX_ROWS):
            return False
        if kernels._lib.timeline is not None:
            return False
        for r in rows:
            if r.source is not None or len(r.want) != 1:
                return False
        T_pad = -(-int(lens.sum()) // PromptGraph.PAD) * PromptGraph.PAD
        if int(lens.max()) < 2 or T_pad > min(PromptGraph.MAX_TOKENS, self.runtime.max_context):
            return False
        if any(self.cache.book.lengths([r.slot for r in rows])):
            return False                                   # a continuation: its keys come from the pages
        # every size of a single prompt may be captured; of the others as many as the engine keeps room for
        return (len(rows), T_pad) in self._prompt_graphs or len(rows) == 1 \
            or len(self._prompt_graphs) < PromptGraph.MAX_GRAPHS - PromptGraph.MAX_TOKENS // PromptGraph.PAD

    def check_status(self) -> None:
        """Raises if a kernel of an earlier step gave up on a bounded wait
        (waits for the device).  Replayed decode steps do not check by
        themselves: the generation loop reads the status word with every
        step's sampled ids, and whoever else replays steps calls this before
        it uses their results."""
        kernels.check_tc_status()

    # ---- generation (see generate.py) ----------------------------------------
    def generate(self, prompts, params=None, **kwargs):
        from .generate import generate
        return generate(self, prompts, params, **kwargs)
