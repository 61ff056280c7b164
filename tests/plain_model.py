"""Plain, slow implementation of the Qwen2.5 dense decoder and of the samplers.

Written from the formulas of the reference engine (paths are relative to the
reference project's root).  The reference cannot be compiled or imported in
this environment (no Rust toolchain, no crate registry), so this file rests on
its formulas alone; every function cites the lines it restates.

Rules of this file: whole sequences only, no cache, one function per part,
explicit masks, nothing imported from the product package.  All math is done
in the dtype of the tensors handed in (float32, or float64 when a test wants a
tighter anchor).
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/models/turbo_generic.rs:41-51 — variance = mean(x^2) over the last
    dim, y = x / sqrt(variance + eps) * weight."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    rms = torch.sqrt(variance + eps)
    return (x / rms) * weight.to(x.dtype)


def rope_tables(head_dim: int, theta: float, n_positions: int, dtype=torch.float32):
    """src/models/turbo_generic.rs:1654-1670 — inv[j] = 1 / theta^(2j/head_dim)
    computed in float32, angle[p, j] = float(p) * inv[j], tables cos/sin
    [n_positions, head_dim/2].  The table itself is always built in float32 (as
    the reference does) and then cast."""
    theta32 = torch.tensor(float(theta), dtype=torch.float32)
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float32) / float(head_dim)
    inv = 1.0 / torch.pow(theta32, exponents)
    pos = torch.arange(n_positions, dtype=torch.float32).reshape(n_positions, 1)
    ang = pos * inv.reshape(1, -1)
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def rope_halved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """src/models/turbo_generic.rs:417-427 — x: [heads, seq, head_dim];
    cos/sin: [seq, head_dim/2].  First half / second half rotation."""
    half = x.shape[-1] // 2
    x0 = x[..., :half]
    x1 = x[..., half:]
    c = cos.unsqueeze(0)
    s = sin.unsqueeze(0)
    r0 = x0 * c - x1 * s
    r1 = x0 * s + x1 * c
    return torch.cat([r0, r1], dim=-1)


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """src/models/turbo_generic.rs:195-204 — kv head g serves q heads
    g*n_rep .. g*n_rep + n_rep - 1.  x: [kv_heads, seq, head_dim]."""
    if n_rep == 1:
        return x
    kvh, s, d = x.shape
    return x.unsqueeze(1).expand(kvh, n_rep, s, d).reshape(kvh * n_rep, s, d)


def attention_mask(seq: int, window: int | None) -> torch.Tensor:
    """src/models/turbo_generic.rs:1937-1948 — True where the score is masked:
    key j after query i.  The sliding window is not in the reference; the rule
    used by this project is: a windowed layer lets query i see keys
    max(0, i - window + 1) .. i."""
    i = torch.arange(seq).reshape(seq, 1)
    j = torch.arange(seq).reshape(1, seq)
    masked = j > i
    if window is not None:
        masked = masked | (j < i - window + 1)
    return masked


def softmax_last_dim(x: torch.Tensor) -> torch.Tensor:
    """src/models/turbo_generic.rs:56-62."""
    m = x.max(dim=-1, keepdim=True).values
    e = torch.exp(x - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention(x, wq, bq, wk, bk, wv, bv, wo, n_heads, n_kv_heads, head_dim, cos, sin, window):
    """src/models/turbo_generic.rs:778-781 (projections), :805-813 (bias after
    the product), :815-817 (head split, head-major features), :832-833 (RoPE on
    q and k), :1620-1631 (GQA expand, scores / sqrt(head_dim), mask with -inf,
    softmax, P·V), :1633-1634 (merge heads, output projection without bias).
    x: [seq, hidden] (already normed)."""
    seq = x.shape[0]
    q = x @ wq.T + bq
    k = x @ wk.T + bk
    v = x @ wv.T + bv
    q = q.reshape(seq, n_heads, head_dim).transpose(0, 1)
    k = k.reshape(seq, n_kv_heads, head_dim).transpose(0, 1)
    v = v.reshape(seq, n_kv_heads, head_dim).transpose(0, 1)
    q = rope_halved(q, cos[:seq], sin[:seq])
    k = rope_halved(k, cos[:seq], sin[:seq])
    n_rep = n_heads // n_kv_heads
    k = repeat_kv(k, n_rep)
    v = repeat_kv(v, n_rep)
    att = (q @ k.transpose(1, 2)) / math.sqrt(head_dim)
    masked = attention_mask(seq, window)
    att = torch.where(masked.unsqueeze(0), torch.full_like(att, float("-inf")), att)
    att = softmax_last_dim(att)
    y = att @ v
    y = y.transpose(0, 1).reshape(seq, n_heads * head_dim)
    return y @ wo.T


def swiglu_mlp(x, w_gate, w_up, w_down):
    """src/models/turbo_generic.rs:105-110 — down(silu(gate x) * (up x))."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (torch.nn.functional.silu(g) * u) @ w_down.T


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------


def layer_is_windowed(cfg: dict, layer: int) -> bool:
    """Not in the reference.  Rule of this project: layer l uses the window iff
    use_sliding_window and l >= max_window_layers."""
    if not cfg.get("use_sliding_window", False):
        return False
    return layer >= int(cfg.get("max_window_layers", cfg["num_hidden_layers"]))


def decoder_logits(cfg: dict, weights: dict, tokens, dtype=torch.float32) -> torch.Tensor:
    """src/models/turbo_generic.rs:1950-1987 — embedding, per layer
    {norm, attention, residual, norm, MLP, residual}, final norm, LM head.
    Returns logits at every position: [seq, vocab].  (The reference keeps the
    last row only; the other rows follow from the same formula.)"""
    w = {k: v.to(dtype) for k, v in weights.items() if v.is_floating_point()}
    n_layers = int(cfg["num_hidden_layers"])
    hidden = int(cfg["hidden_size"])
    n_heads = int(cfg["num_attention_heads"])
    n_kv = int(cfg.get("num_key_value_heads", n_heads))
    head_dim = int(cfg.get("head_dim", hidden // n_heads))
    eps = float(cfg["rms_norm_eps"])
    theta = float(cfg["rope_theta"])
    toks = torch.as_tensor(tokens, dtype=torch.long)
    seq = toks.shape[0]
    cos, sin = rope_tables(head_dim, theta, seq, dtype)
    h = w["model.embed_tokens.weight"][toks]
    for i in range(n_layers):
        p = f"model.layers.{i}"
        window = int(cfg["sliding_window"]) if layer_is_windowed(cfg, i) else None
        a = rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
        attn = attention(
            a,
            w[f"{p}.self_attn.q_proj.weight"], w[f"{p}.self_attn.q_proj.bias"],
            w[f"{p}.self_attn.k_proj.weight"], w[f"{p}.self_attn.k_proj.bias"],
            w[f"{p}.self_attn.v_proj.weight"], w[f"{p}.self_attn.v_proj.bias"],
            w[f"{p}.self_attn.o_proj.weight"],
            n_heads, n_kv, head_dim, cos, sin, window,
        )
        h = attn + h
        m = rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)
        h = swiglu_mlp(m, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                       w[f"{p}.mlp.down_proj.weight"]) + h
    n = rms_norm(h, w["model.norm.weight"], eps)
    # src/models/turbo_generic.rs:2079-2084 — lm_head.weight if present, else
    # the embedding matrix.
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return n @ head.T


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------


def apply_repeat_penalty(logits: torch.Tensor, generated: list[int], penalty: float) -> torch.Tensor:
    """src/engine.rs:403-419 — for every generated token (once per
    occurrence, the prompt excluded): l > 0 ? l / p : l * p."""
    out = logits.clone()
    if penalty == 1.0:
        return out
    for t in generated:
        if 0 <= t < out.shape[0]:
            s = out[t]
            out[t] = s / penalty if s > 0 else s * penalty
    return out


def greedy(logits: torch.Tensor) -> int:
    """src/engine.rs:353-354 — temperature <= 0 selects arg-max.  Ties go to
    the lowest token id (rule of this project)."""
    m = logits.max()
    return int(torch.nonzero(logits == m)[0, 0])


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """src/engine.rs:353-360 — temperature > 0 selects top-k then top-p on
    softmax(logits / temperature).  The sampler itself lives outside the
    reference's tree, so the details are this project's:
      * top-k keeps every token whose logit is >= the k-th largest logit
        (0 or >= vocab: off);
      * top-p, applied to what top-k kept, walks the kept tokens by
        descending probability and keeps every token whose probability is >=
        that of the token at which the running mass first reaches top_p times
        the kept mass (>= 1: off);
      * the draw walks the kept tokens in token-id order and returns the
        first token whose running mass exceeds u times the kept mass.
    Probabilities are float32 exponentials; masses are summed in float64."""
    if temperature <= 0.0:
        return greedy(logits)
    l32 = logits.to(torch.float32)
    m = l32.max()
    p = torch.exp((l32 - m) / torch.tensor(temperature, dtype=torch.float32))
    keep = torch.ones_like(p, dtype=torch.bool)
    vocab = p.shape[0]
    if 0 < top_k < vocab:
        kth = torch.sort(l32, descending=True).values[top_k - 1]
        keep &= l32 >= kth
    if top_p < 1.0:
        pk = torch.where(keep, p, torch.zeros_like(p))
        order = torch.sort(pk, descending=True, stable=True)
        cum = torch.cumsum(order.values.to(torch.float64), 0)
        total = cum[-1]
        first = int(torch.nonzero(cum >= top_p * total)[0, 0])
        cut = order.values[first]
        keep &= p >= cut
    pk = torch.where(keep, p, torch.zeros_like(p)).to(torch.float64)
    cum = torch.cumsum(pk, 0)
    target = u * cum[-1]
    hit = torch.nonzero(cum > target)
    return int(hit[0, 0]) if hit.numel() else int(torch.nonzero(keep)[-1, 0])


def generate(cfg: dict, weights: dict, prompt: list[int], max_tokens: int, *, temperature=0.0,
             top_k=0, top_p=1.0, repeat_penalty=1.0, uniforms=None, stop=()) -> list[int]:
    """src/engine.rs:333-446 — the loop: sample from the prompt's last logits,
    stop before emitting a stop token, otherwise emit, run the model on the
    sequence so far, penalise, sample.  Recomputes the whole sequence each
    time.  `uniforms[i]` is the draw used for the i-th sampled token."""
    seq = list(prompt)
    out: list[int] = []
    for i in range(max_tokens):
        logits = decoder_logits(cfg, weights, seq)[-1]
        logits = apply_repeat_penalty(logits, out, repeat_penalty)
        u = uniforms[i] if uniforms is not None else 0.0
        nxt = sample(logits, temperature, top_k, top_p, u)
        if nxt in stop:
            break
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------
# reading a model folder (independent of the product's loader)
# --------------------------------------------------------------------------

_DT = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
       "I32": (torch.int32, 4), "I64": (torch.int64, 8)}


def read_model_folder(folder: str):
    """config.json as a plain dict and every tensor of model.safetensors as
    float32 (integers kept).  File layout: 8-byte little-endian header length,
    JSON header {name: {dtype, shape, data_offsets}}, raw data."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _DT[meta["dtype"]]
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(blob[a:b]), dtype=dt).reshape(meta["shape"])
        tensors[name] = t.to(torch.float32) if t.is_floating_point() else t
    return cfg, tensors
