"""Python entry point of the attention kernel (csrc/attention.cu)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream, tc_status_word

MAX_HEAD_DIM = 256
NOT_SUPPORTED = 801     # cudaErrorNotSupported: a specialised kernel declines the shape
USE_TC_ATTENTION = True  # prompts: the tcgen05 kernel (csrc/flash_prefill_tc.cu) before the mma.sync one


def check_head_geometry(n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Raises for head sizes the attention kernels do not take."""
    if head_dim % 16 or not 16 <= head_dim <= MAX_HEAD_DIM:
        raise KernelError(f"attention: head_dim {head_dim} must be a multiple of 16 between 16 and {MAX_HEAD_DIM}")
    if n_kv_heads <= 0 or n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} heads cannot be shared among {n_kv_heads} key/value heads")
    if n_kv_heads > 65535:
        raise KernelError(f"attention: more than 65535 key/value heads ({n_kv_heads})")


def plan_splits(n_tokens: int, n_kv_heads: int, max_keys: int, sm_count: int) -> int:
    """Number of splits of the key range for a step: one while the grid fills
    the GPU or the key ranges are short, else as many as fill the GPU in one
    wave, with at least 128 keys per split of the longest range.  (Each
    token cuts its own range into that many equal parts.)"""
    blocks = n_tokens * n_kv_heads
    resident = 2 * sm_count                    # blocks of the decode kernel that run at once
    if blocks >= resident or max_keys <= 256:
        return 1
    # fill the GPU once: a grid a little over a whole number of waves wastes most of its last wave
    return max(1, min(resident // blocks, -(-max_keys // 128), 64))


def split_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_tokens * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attention(q: torch.Tensor, out: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
              tok_pos: torch.Tensor, tok_seq: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
              window: Optional[int], scale: Optional[float] = None,
              k_packed: Optional[torch.Tensor] = None, v_packed: Optional[torch.Tensor] = None,
              k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
              block_table: Optional[torch.Tensor] = None, table_width: int = 0, ring_pages: int = 0,
              page_tokens: int = 64, n_splits: int = 1,
              scratch: Optional[torch.Tensor] = None, use_flash: bool = True):
    """out[t, h] = softmax(q[t, h] · K / sqrt(head_dim)) · V over the keys
    max(0, pos-window+1) .. pos of the token's sequence.  q/out [T, nh*hd].
    Keys and values come from the step's packed rows (k_packed/v_packed
    [T, nkv*hd]; every sequence must then start at position 0 or carry its
    whole history in the step) or from the paged cache."""
    check_head_geometry(n_heads, n_kv_heads, head_dim)
    T = q.shape[0]
    if q.shape[1] != n_heads * head_dim or out.shape != q.shape or out.dtype != q.dtype:
        raise KernelError("attention: q and out must be [T, n_heads*head_dim] of one dtype")
    packed = k_packed is not None
    if packed:
        if v_packed is None or k_packed.dtype != q.dtype or k_packed.shape != (T, n_kv_heads * head_dim):
            raise KernelError("attention: packed keys/values must be [T, n_kv_heads*head_dim] of q's dtype")
    else:
        if k_pages is None or v_pages is None or block_table is None or k_pages.dtype != q.dtype:
            raise KernelError("attention: no key/value source of q's dtype was given")
        if tuple(k_pages.shape[1:]) != (n_kv_heads, page_tokens, head_dim):
            raise KernelError(f"attention: cache pages have shape {tuple(k_pages.shape)}")
    part_acc = part_ml = None
    if n_splits > 1:
        need = split_scratch_floats(T, n_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: {n_splits} splits need {need} float32 of scratch")
        n_acc = T * n_heads * n_splits * head_dim
        part_acc, part_ml = scratch[:n_acc], scratch[n_acc:need]
    need_contiguous(q=q, out=out, k_packed=k_packed, v_packed=v_packed, k_pages=k_pages, v_pages=v_pages,
                    block_table=block_table)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    n_seqs = cu_seqlens.shape[0] - 1
    if q.dtype == torch.bfloat16 and use_flash and USE_TC_ATTENTION and T > n_seqs:
        # prompts on the tcgen05 tensor cores (128-query tiles, S and P·V in tensor memory)
        st = core().tq_flash_prefill_tc(
            ptr(q), ptr(k_packed), ptr(v_packed), ptr(k_pages), ptr(v_pages),
            0 if k_pages is None else k_pages.shape[0], ptr(block_table), table_width, ring_pages, page_tokens,
            ptr(cu_seqlens), ptr(start_pos), n_seqs, T, int(window or 0), float(scale), ptr(out), n_heads,
            n_kv_heads, head_dim, ptr(tc_status_word(q.device)), stream())
        if st != NOT_SUPPORTED:
            check(st, "flash_prefill_tc")
            return out
    if q.dtype == torch.bfloat16 and use_flash and T > n_seqs:
        # prompts (some sequence brings several tokens): the tensor-core kernel with 64-query tiles
        st = core().tq_flash_prefill(
            ptr(q), ptr(k_packed), ptr(v_packed), ptr(k_pages), ptr(v_pages), ptr(block_table), table_width,
            ring_pages, page_tokens, ptr(cu_seqlens), ptr(start_pos), n_seqs, T, int(window or 0), float(scale),
            ptr(out), n_heads, n_kv_heads, head_dim, stream())
        if st != NOT_SUPPORTED:
            check(st, "flash_prefill")
            return out
    if not packed and q.dtype == torch.bfloat16 and use_flash:
        # the bandwidth-built kernel for the cache; it declines shapes outside its reach
        st = core().tq_flash_decode(
            ptr(q), ptr(k_pages), ptr(v_pages), ptr(block_table), table_width, ring_pages, page_tokens,
            ptr(tok_pos), ptr(tok_seq), int(window or 0), float(scale), ptr(out), ptr(part_acc), ptr(part_ml), T,
            n_heads, n_kv_heads, head_dim, n_splits, stream())
        if st != NOT_SUPPORTED:
            check(st, "flash_decode")
            if n_splits > 1:
                check(core().tq_attention_merge(ptr(part_acc), ptr(part_ml), ptr(out), dtype_code(out), T, n_heads,
                                                head_dim, n_splits, stream()), "attention_merge")
            return out
    check(core().tq_attention(
        ptr(q), dtype_code(q), ptr(k_packed), ptr(v_packed), ptr(k_pages), ptr(v_pages), ptr(block_table),
        table_width, ring_pages, page_tokens, ptr(tok_pos), ptr(tok_seq), ptr(cu_seqlens), ptr(start_pos),
        int(window or 0), float(scale), ptr(out), ptr(part_acc), ptr(part_ml), T, n_heads, n_kv_heads, head_dim,
        n_splits, stream()), "attention", 2 if n_splits > 1 else 1)
    return out
