"""Shared helpers of the tests: the tiny configurations, model folders made
in temporary directories, the plain implementation as oracle, tolerances."""
from __future__ import annotations

import os

import torch

import plain_model

# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "float32",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "sliding_window": None, "max_window_layers": 2,
    "max_position_embeddings": 512,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "float32",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 200, "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 16, "max_window_layers": 1,
    "max_position_embeddings": 1024,
}
TINY = {"a": TINY_A, "b": TINY_B}

_folders: dict = {}
_plain_cache: dict = {}


def model_folder(tmp_root, name: str, dtype: str, seed: int = 1234) -> str:
    """A model folder with random weights for tiny config `name`, stored in
    `dtype`; made once per test session."""
    from tq_kv_b200.weights import write_model_folder
    key = (name, dtype, seed)
    if key not in _folders:
        cfg = dict(TINY[name])
        cfg["torch_dtype"] = dtype
        folder = os.path.join(str(tmp_root), f"tiny_{name}_{dtype}_{seed}")
        write_model_folder(cfg, folder, seed)
        _folders[key] = folder
    return _folders[key]


def plain_logits(folder: str, tokens: list[int], dtype=torch.float32) -> torch.Tensor:
    """Logits of the plain implementation at every position of `tokens`."""
    key = (folder, tuple(tokens), dtype)
    if key not in _plain_cache:
        cfg, w = plain_model.read_model_folder(folder)
        _plain_cache[key] = plain_model.decoder_logits(cfg, w, tokens, dtype).to(torch.float32)
    return _plain_cache[key]


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# Tolerances (max |difference| of logits), relative to max(1, max |logit|):
#   float32 engine vs plain float32: rounding of different summation orders;
#   bfloat16 engine vs plain float32 on the same (bfloat16-valued) weights:
#   activations rounded to 8 bits of mantissa between the parts.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float32)
    want = want.to(torch.float32)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: max |diff| {err:.3e} > {TOL[dtype] * scale:.3e} ({dtype})"
