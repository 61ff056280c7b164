"""Rotary position encoding, rotate-half layout.

Reference: tables — src/models/turbo_generic.rs:1654-1670: inv[j] =
1 / theta^(2j / rotary_dim) in float32, angle[p, j] = float32(p) * inv[j],
cos and sin of the angles, [positions, rotary_dim / 2] float32; application —
:417-427 (first half / second half) at rows `index_pos .. index_pos + s`
(:746-768).  Keys are cached after the rotation (:832-833, :1606-1618).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import PositionEncoding, Runtime, StepContext


class RotaryHalved(PositionEncoding):
    padded_rows_ok = True               # rows at or past their sequence's new length are not cached

    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(self.params["head_dim"])
        self.rotary_dim = int(self.params["rotary_dim"])
        self.theta = float(self.params["theta"])
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def table_key(self):
        return ("rotary_halved", self.rotary_dim, self.theta)

    def prepare(self, runtime: Runtime, shared: Optional[dict] = None) -> None:
        """Tables are computed once per (rotary_dim, theta) and shared by the
        layers of a model through `shared`.  They are built on the host in
        float32, as the reference builds them, then copied to the device."""
        key = (self.table_key(), runtime.max_context, str(runtime.device))
        if shared is not None and key in shared:
            self.cos, self.sin = shared[key]
            return
        theta = torch.tensor(self.theta, dtype=torch.float32)
        expo = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / float(self.rotary_dim)
        inv = 1.0 / torch.pow(theta, expo)
        pos = torch.arange(runtime.max_context, dtype=torch.float32).reshape(-1, 1)
        ang = pos * inv.reshape(1, -1)
        self.cos = torch.cos(ang).contiguous().to(runtime.device)
        self.sin = torch.sin(ang).contiguous().to(runtime.device)
        if shared is not None:
            shared[key] = (self.cos, self.sin)

    clears_input = True          # encode_and_store(..., clear_input=True) leaves zeros in qkv

    def encode_and_store(self, qkv, bias, ctx: StepContext, *, n_heads, n_kv_heads, head_dim, q_out, k_out, v_out,
                         clear_input=False):
        b = ctx.batch
        kv = ctx.kv
        write = kv is not None and kv.writes
        table, width = (kv.block_table, kv.table_width) if write else (None, 0)
        kernels.qkv_rope_cache(
            qkv, bias, self.cos, self.sin, b.tok_pos, b.tok_seq, b.new_lens, q_out,
            n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, rotary_dim=self.rotary_dim,
            k_out=k_out, v_out=v_out,
            k_pages=kv.k_pages if write else None, v_pages=kv.v_pages if write else None,
            block_table=table, table_width=width, ring_pages=kv.ring_pages if write else 0,
            page_tokens=kv.page_tokens if kv is not None else 64, clear_input=clear_input)
