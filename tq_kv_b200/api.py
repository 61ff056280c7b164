"""The Python entry point: `load()` a model, then `Engine.generate()`.

    import tq_kv_b200 as tq
    engine = tq.load("path/to/model_folder")                  # config.json + *.safetensors
    engine = tq.load("tiny-a", random_weights=True, seed=1)   # a named shape with random weights
    out = engine.generate([[1, 2, 3], [4, 5]], tq.GenerationParams(max_tokens=16, temperature=0.0))
    out[0].tokens, out[0].finish_reason

`EngineBuilder` offers the same in the reference's fluent manner
(src/engine.rs:123-205: Engine::builder().model(..).build()).
"""
from __future__ import annotations

import os
from typing import Optional

from .config import named_shape, shape_names
from .engine import Engine


def load(model: str, *, dtype: str = "bfloat16", device: str = "cuda:0", random_weights: bool = False, seed: int = 0,
         max_batch: int = 8, max_context: Optional[int] = None, max_tokens: Optional[int] = None,
         window_chunk: int = 64) -> Engine:
    """An engine for `model`: a folder with config.json and safetensors files,
    or — with `random_weights` — a folder's config.json or the name of a shape
    (`tq_kv_b200.shape_names()`).  The cache holds `max_batch` sequences of
    `max_context` tokens unless `max_tokens` (tokens held together) is given.
    `window_chunk` is the most tokens one step may add to a sequence it
    continues in a layer with a sliding window."""
    if random_weights:
        if os.path.isdir(model) or os.path.isfile(model):
            from .config import read_config_json
            cfg = read_config_json(model)
        else:
            cfg = named_shape(model)
        return Engine.from_random(cfg, seed, dtype=dtype, device=device, max_tokens=max_tokens, max_slots=max_batch,
                                  max_context=max_context, window_chunk=window_chunk)
    if not os.path.isdir(model):
        hint = f" ('{model}' is a shape name: pass random_weights=True)" if model in shape_names() else ""
        raise FileNotFoundError(f"model folder '{model}' does not exist{hint}")
    return Engine.from_folder(model, dtype=dtype, device=device, max_tokens=max_tokens, max_slots=max_batch,
                              max_context=max_context, window_chunk=window_chunk)


class EngineBuilder:
    """Fluent construction, after src/engine.rs:132-205."""

    def __init__(self):
        self._kw: dict = {}
        self._model: Optional[str] = None

    def model(self, path: str) -> "EngineBuilder":
        self._model = path
        return self

    def dtype(self, dtype: str) -> "EngineBuilder":
        self._kw["dtype"] = dtype
        return self

    def device(self, device: str) -> "EngineBuilder":
        self._kw["device"] = device
        return self

    def random_weights(self, seed: int = 0) -> "EngineBuilder":
        self._kw.update(random_weights=True, seed=seed)
        return self

    def max_batch(self, n: int) -> "EngineBuilder":
        self._kw["max_batch"] = n
        return self

    def max_context(self, n: int) -> "EngineBuilder":
        self._kw["max_context"] = n
        return self

    def build(self) -> Engine:
        if self._model is None:
            raise ValueError("EngineBuilder: no model was given")
        return load(self._model, **self._kw)
