"""Python entry points of the memory-bound kernels (csrc/elementwise.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t] = float32(table[tokens[t]]).  tokens int32 [T]; table [V, H]
    float32 or bfloat16; out float32 [T, H].  `status` (int32 [1]) gets bit 0
    set if a token id lies outside the table."""
    T = tokens.shape[0]
    V, H = table.shape
    if tokens.dtype != torch.int32 or out.dtype != torch.float32 or tuple(out.shape) != (T, H):
        raise KernelError("embed: tokens must be int32 [T] and out float32 [T, H]")
    need_contiguous(tokens=tokens, table=table, out=out)
    check(core().tq_embed(ptr(tokens), ptr(table), dtype_code(table), ptr(out), T, H, V, ptr(status), stream()),
          "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None):
    """out[r] = x[rows[r] or r] / sqrt(mean(x^2) + eps) * weight.  x float32
    [*, H]; weight float32 [H]; out float32 or bfloat16 [R, H]."""
    H = x.shape[-1]
    R = out.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.shape[0] != H or out.shape[-1] != H:
        raise KernelError("rmsnorm: x and weight must be float32 with matching width")
    if rows is None and x.shape[0] != R:
        raise KernelError("rmsnorm: out must have as many rows as x when no rows are selected")
    if rows is not None and (rows.dtype != torch.int32 or rows.shape[0] != R):
        raise KernelError("rmsnorm: rows must be int32 [R]")
    need_contiguous(x=x, weight=weight, out=out, rows=rows)
    check(core().tq_rmsnorm(ptr(x), ptr(weight), ptr(out), dtype_code(out), ptr(rows), R, H, float(eps), stream()),
          "rmsnorm")
    return out


def qkv_rope_cache(qkv, bias, cos, sin, tok_pos, tok_seq, new_lens, q_out, *, n_heads, n_kv_heads, head_dim,
                   rotary_dim, k_out=None, v_out=None, k_pages=None, v_pages=None, block_table=None,
                   table_width=0, ring_pages=0, page_tokens=64, clear_input=False):
    """Bias, rotary encoding of q and k, head split, cache append (see
    csrc/elementwise.cu).  qkv [T, (nh+2nkv)*hd]; cos/sin float32
    [positions, rotary_dim/2]; q_out/k_out/v_out and the pages share one dtype.
    With `clear_input` the kernel leaves zeros in the rows of qkv it has read."""
    T = qkv.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv_rope_cache: qkv has width {qkv.shape[1]}, expected {width}")
    if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
        raise KernelError(f"qkv_rope_cache: rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2:
        raise KernelError("qkv_rope_cache: cos/sin must be float32 [positions, rotary_dim/2]")
    for t in (k_out, v_out, k_pages, v_pages):
        if t is not None and t.dtype != q_out.dtype:
            raise KernelError("qkv_rope_cache: outputs and cache pages must share one dtype")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != width):
        raise KernelError("qkv_rope_cache: bias must be float32 of the qkv width")
    need_contiguous(qkv=qkv, bias=bias, cos=cos, sin=sin, q_out=q_out, k_out=k_out, v_out=v_out, k_pages=k_pages,
                    v_pages=v_pages)
    check(core().tq_qkv_rope_cache(
        ptr(qkv), dtype_code(qkv), ptr(bias), ptr(cos), ptr(sin), ptr(tok_pos), ptr(tok_seq), ptr(new_lens),
        ptr(block_table), table_width, ring_pages, page_tokens, ptr(q_out), ptr(k_out), ptr(v_out), ptr(k_pages),
        ptr(v_pages), dtype_code(q_out), T, n_heads, n_kv_heads, head_dim, rotary_dim, int(clear_input), stream()),
        "qkv_rope_cache")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor):
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    T, two_i = gate_up.shape
    I = two_i // 2
    if two_i != 2 * I or tuple(out.shape) != (T, I):
        raise KernelError("swiglu: gate_up must be [T, 2I] and out [T, I]")
    need_contiguous(gate_up=gate_up, out=out)
    check(core().tq_swiglu(ptr(gate_up), dtype_code(gate_up), ptr(out), dtype_code(out), T, I, stream()), "swiglu")
    return out


def add_into(acc: torch.Tensor, x: torch.Tensor):
    """acc += float32(x), acc float32."""
    if acc.dtype != torch.float32 or acc.shape != x.shape:
        raise KernelError("add_into: acc must be float32 and of x's shape")
    need_contiguous(acc=acc, x=x)
    check(core().tq_add_into(ptr(acc), ptr(x), dtype_code(x), acc.numel(), stream()), "add_into")
    return acc


def select_tokens(tokens: torch.Tensor, source_rows: torch.Tensor, sampled: torch.Tensor):
    """tokens[i] = sampled[source_rows[i]] where source_rows[i] >= 0; other
    entries keep the id the host put there.  All int32, on the device: the
    token a sequence decodes next can be the one the sampler just chose,
    without a trip through the host."""
    n = tokens.shape[0]
    for name, t in (("tokens", tokens), ("source_rows", source_rows), ("sampled", sampled)):
        if t.dtype != torch.int32:
            raise KernelError(f"select_tokens: {name} must be int32")
    if source_rows.shape[0] < n:
        raise KernelError("select_tokens: one source row per token")
    need_contiguous(tokens=tokens, source_rows=source_rows, sampled=sampled)
    check(core().tq_select_tokens(ptr(tokens), ptr(source_rows), ptr(sampled), n, stream()), "select_tokens")
    return tokens


def random_fill(out: torch.Tensor, key: int, std: float, offset: float = 0.0):
    """out[i] = offset + std * z(key, i) with z standard normal from the
    counter-based generator of csrc/random_fill.cu (float32 or bfloat16 out)."""
    need_contiguous(out=out)
    check(core().tq_random_fill(ptr(out), dtype_code(out), out.numel(), int(key) & ((1 << 64) - 1), float(std),
                                float(offset), stream()), "random_fill")
    return out
