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


TINY_C = {          # a third configuration; planted_model() plants one decisive key into its first layer
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "float32",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48,
    "intermediate_size": 208, "vocab_size": 520, "rope_theta": 50000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 0,
    "max_position_embeddings": 1024,
}
TINY["c"] = TINY_C
PLANT_KEY_TOKEN, PLANT_QUERY_TOKEN = 7, 11


def planted_model(tmp_root, dtype: str, windowed: bool, seed: int = 77) -> str:
    """Tiny C (every layer windowed, or none) with random weights in which one
    key decides: in layer 0, query head 4 of token PLANT_QUERY_TOKEN scores
    about 12 against the key of token PLANT_KEY_TOKEN and about 1 against
    every other key, wherever the two stand (the planted components sit in the
    head's slowest rotary pair, which turns by less than 0.01 rad over a
    thousand positions); that key's value is scaled up, so that the logits at
    the query's place change wholly with whether the key is seen.  A kernel
    that drops this key, sees it from one place too far, or reads its slot of
    the cache wrongly is then off by the size of the logits, in bfloat16 too."""
    from tq_kv_b200.weights import write_model_folder, write_safetensors
    key = ("planted", dtype, windowed, seed)
    if key in _folders:
        return _folders[key]
    cfg = {**TINY_C, "torch_dtype": dtype, "use_sliding_window": windowed}
    plain = os.path.join(str(tmp_root), f"tiny_c_{dtype}_{windowed}_{seed}")
    write_model_folder(cfg, plain, seed)
    _, w = plain_model.read_model_folder(plain)
    hd, nh, nkv, c = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"], 9.0
    hq = 4
    g = hq // (nh // nkv)
    d = hd // 2 - 1                                   # the slowest pair is (hd/2 - 1, hd - 1)
    E, ln = w["model.embed_tokens.weight"].float(), w["model.layers.0.input_layernorm.weight"].float()
    a = {t: plain_model.rms_norm(E[t], ln, cfg["rms_norm_eps"]) for t in (PLANT_KEY_TOKEN, PLANT_QUERY_TOKEN)}
    out = {n: t.clone() for n, t in w.items()}
    p = "model.layers.0.self_attn."

    def put(name, row, values):
        t = out[name].float()
        t[row] = values
        out[name] = t.to(w[name].dtype)

    ak, aq = a[PLANT_KEY_TOKEN], a[PLANT_QUERY_TOKEN]
    for row_k, row_q in ((g * hd + d, hq * hd + d), (g * hd + d + hd // 2, hq * hd + d + hd // 2)):
        put(p + "k_proj.weight", row_k, c * ak / (ak @ ak) if row_k % hd == d else torch.zeros_like(ak))
        put(p + "q_proj.weight", row_q, c * aq / (aq @ aq) if row_q % hd == d else torch.zeros_like(aq))
        put(p + "k_proj.bias", row_k, 0.0)
        put(p + "q_proj.bias", row_q, 0.0)
    t = out[p + "v_proj.weight"].float()
    t[g * hd:(g + 1) * hd] *= 8.0
    out[p + "v_proj.weight"] = t.to(w[p + "v_proj.weight"].dtype)
    t = out[p + "o_proj.weight"].float()
    t[:, hq * hd:(hq + 1) * hd] *= 4.0
    out[p + "o_proj.weight"] = t.to(w[p + "o_proj.weight"].dtype)
    folder = plain + "_planted"
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), [(n, t.dtype, tuple(t.shape)) for n, t in out.items()],
                      list(out.items()), metadata={"format": "pt"})
    with open(os.path.join(plain, "config.json")) as f_in, open(os.path.join(folder, "config.json"), "w") as f_out:
        f_out.write(f_in.read())
    _folders[key] = folder
    return folder


def planted_tokens(n: int, key_at: int, query_at: list[int], seed: int) -> list[int]:
    """n random tokens of tiny C's vocabulary without the two planted ones,
    then the key token at `key_at` and the query token at each of `query_at`."""
    toks = [t for t in random_tokens(2 * n, TINY_C["vocab_size"], seed)
            if t not in (PLANT_KEY_TOKEN, PLANT_QUERY_TOKEN)][:n]
    toks[key_at] = PLANT_KEY_TOKEN
    for q in query_at:
        toks[q] = PLANT_QUERY_TOKEN
    return toks


def random_weights(cfg: dict, seed: int, device="cuda"):
    """The tensors that `Engine.from_random(cfg, seed)` holds, by name, made on
    `device` in the configuration's stored dtype: the plain implementation can
    then be compared with such an engine without a trip through a file."""
    from tq_kv_b200.config import spec_from_config_dict
    from tq_kv_b200.engine import DecoderModel
    from tq_kv_b200.weights.random_init import random_tensors, storage_dtype
    _, _, spec = spec_from_config_dict(cfg)
    specs = DecoderModel(spec).weight_specs().values()
    return dict(random_tensors(specs, seed, storage_dtype(cfg.get("torch_dtype", "bfloat16")), device))


def plain_logits_on(device, cfg: dict, weights: dict, tokens: list[int]) -> torch.Tensor:
    """The plain implementation run on `device` in float32 (true float32
    products: TF32 stays off), for models too large for the CPU in a test."""
    assert not torch.backends.cuda.matmul.allow_tf32
    with torch.device(device):
        return plain_model.decoder_logits(cfg, weights, tokens, torch.float32).to("cpu", torch.float32)


# Tolerances: max |difference| of logits relative to max |logit| of the plain implementation (no floor: the tiny
# models' logits lie within +-0.6, and a floor of 1 would let a tenth of that range pass).
#   float32 engine vs plain float32: rounding of different summation orders;
#   bfloat16 engine vs plain float32 on the same (bfloat16-valued) weights: activations rounded to 8 bits of
#   mantissa between the parts.  The bounds are two to four times the largest error seen over the test suite
#   (7e-6 and 1.4e-2, the latter in 60 decode steps at the 7B layer sizes); pytest prints the largest ratios
#   seen at the end of a run (conftest.py).
TOL = {"float32": 3e-5, "bfloat16": 3e-2}
worst: dict = {}          # (dtype) -> (ratio, what)


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", tol: float | None = None) -> None:
    got = got.detach().to("cpu", torch.float32)
    want = want.to("cpu", torch.float32)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    ratio = err / scale if scale > 0 else err
    if ratio > worst.get(dtype, (0.0, ""))[0]:
        worst[dtype] = (ratio, what)
    bound = TOL[dtype] if tol is None else tol
    assert ratio <= bound, f"{what}: max |diff| {err:.3e} is {ratio:.3e} of max |logit| {scale:.3e} > {bound:.1e} ({dtype})"
