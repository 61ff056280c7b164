"""Grouped-query attention with optional q/k/v bias, a position encoding part
and an optional sliding window.

Reference: src/models/turbo_generic.rs:778-781 (three projections, here one
product with the concatenated weight), :805-813 (bias after the product, used
iff the tensors exist — here a parameter), :815-817 (head-major split),
:832-833 (position encoding of q and k), :1606-1635 (cache, grouped heads,
scores / sqrt(head_dim), causal mask, softmax, P·V, output projection without
bias), :1969 (residual sum).  The window is this project's rule: the query at
position p sees keys max(0, p - window + 1) .. p.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..cache import PAGE_TOKENS, KVRequest, ring_pages_for
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector
from .registry import make_part


class GQAttention(Mixer):
    takes_pending_norm = True           # x goes to kernels.linear only
    padded_rows_ok = True               # causal: no row sees a later one; the rotary kernel caches real rows only
    ZERO_BUFFER_ROWS = 64               # decode steps of up to this many rows use the shared q/k/v buffer

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p["qkv_bias"])
        self.out_bias = bool(p.get("out_bias", False))
        self.window: Optional[int] = p.get("window")
        self.names = dict(p.get("names", {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}))
        kernels.check_head_geometry(self.n_heads, self.n_kv_heads, self.head_dim)
        self.position = make_part(p["position"])
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.window_chunk = 1

    # ---- weights ----------------------------------------------------------
    def _n(self, which: str, leaf: str) -> str:
        return f"{self.prefix}{self.names[which]}.{leaf}"

    def weight_specs(self):
        specs = [
            WeightSpec(self._n("q", "weight"), (self.q_width, self.hidden), "matrix"),
            WeightSpec(self._n("k", "weight"), (self.kv_width, self.hidden), "matrix"),
            WeightSpec(self._n("v", "weight"), (self.kv_width, self.hidden), "matrix"),
            WeightSpec(self._n("o", "weight"), (self.hidden, self.q_width), "matrix"),
        ]
        if self.qkv_bias:
            specs += [WeightSpec(self._n("q", "bias"), (self.q_width,), "bias"),
                      WeightSpec(self._n("k", "bias"), (self.kv_width,), "bias"),
                      WeightSpec(self._n("v", "bias"), (self.kv_width,), "bias")]
        if self.out_bias:
            specs.append(WeightSpec(self._n("o", "bias"), (self.hidden,), "bias"))
        return specs

    def bind(self, tensors, runtime: Runtime, shared: Optional[dict] = None):
        ws = [tensors[self._n(x, "weight")] for x in "qkv"]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()       # one product for q, k and v
        self.w_o = tensors[self._n("o", "weight")].contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([float32_vector(tensors[self._n(x, "bias")]) for x in "qkv"]).contiguous()
        if self.out_bias:
            self.b_o = float32_vector(tensors[self._n("o", "bias")])
        self.window_chunk = runtime.window_chunk
        key = ("qkv kept zero", self.q_width + 2 * self.kv_width, str(runtime.device))
        store = shared if shared is not None else {}
        if key not in store:                               # one buffer for all layers of this width, and its flag
            store[key] = (torch.zeros((self.ZERO_BUFFER_ROWS, self.q_width + 2 * self.kv_width),
                                      dtype=torch.float32, device=runtime.device), [False])
        self._qkv_zero = store[key]
        self.position.bind(tensors, runtime, shared)      # a position encoding may have tensors of its own
        self.position.prepare(runtime, shared)

    # ---- cache ------------------------------------------------------------
    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def _use_packed(self, start_pos, step_lens, owns_cache) -> bool:
        """Prompts that start at position 0 and own their cache attend over
        the step's own keys; everything else reads the cache."""
        return owns_cache and all(s == 0 for s in start_pos) and any(n > 1 for n in step_lens)

    def check_step(self, start_pos, step_lens, owns_cache):
        if self.window is None or self._use_packed(start_pos, step_lens, owns_cache):
            return
        ring_tokens = ring_pages_for(self.window, self.window_chunk - 1) * PAGE_TOKENS
        longest = max(step_lens)
        if longest > ring_tokens - self.window + 1:
            raise kernels.KernelError(
                f"a layer with a window of {self.window} keeps {ring_tokens} keys per sequence and cannot continue "
                f"a sequence by {longest} tokens in one step (at most {ring_tokens - self.window + 1}; the engine's "
                f"window_chunk option sets this)")

    # ---- one step -----------------------------------------------------------
    def forward(self, x, ctx: StepContext, residual):
        b, kv, dev = ctx.batch, ctx.kv, x.device
        T = x.shape[0]
        act = ctx.runtime.act_dtype
        owns = kv is not None and kv.writes
        packed = self._use_packed(b.host_start, b.host_lens, owns)
        # Where a decode step's q/k/v product adds shares of K into its result, the result must start at zero.
        # Instead of clearing it before every product, the layers share one buffer that is zero between uses:
        # the rotary kernel, which alone reads it, leaves zeros behind.
        kept_zero = (T <= self.ZERO_BUFFER_ROWS and act == torch.bfloat16
                     and getattr(self.position, "clears_input", False)
                     and kernels.product_adds_shares(T, self.w_qkv, isinstance(x, kernels.PendingNorm)))
        if kept_zero:
            buf, dirty = self._qkv_zero
            if dirty[0]:                                   # a step failed between the product and the rotary kernel
                buf.zero_()
            dirty[0] = True
            qkv = kernels.linear(x, self.w_qkv, out=buf[:T], accumulate=True)
        else:
            qkv = kernels.linear(x, self.w_qkv, out_dtype=torch.float32)
        kernels.mark("qkv")
        q = torch.empty((T, self.q_width), dtype=act, device=dev)
        k = torch.empty((T, self.kv_width), dtype=act, device=dev) if packed else None
        v = torch.empty((T, self.kv_width), dtype=act, device=dev) if packed else None
        extra = {"clear_input": True} if kept_zero else {}
        self.position.encode_and_store(qkv, self.b_qkv, ctx, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                                       head_dim=self.head_dim, q_out=q, k_out=k, v_out=v, **extra)
        if kept_zero:
            self._qkv_zero[1][0] = False
        kernels.mark("rotary")
        out = torch.empty_like(q)
        common = dict(n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                      tok_pos=b.tok_pos, tok_seq=b.tok_seq, cu_seqlens=b.cu_seqlens, start_pos=b.start_pos,
                      window=self.window)
        if packed:
            kernels.attention(q, out, k_packed=k, v_packed=v, **common)
        else:
            max_keys = b.max_new_len if self.window is None else min(b.max_new_len, self.window)
            n_splits = kernels.plan_splits(T, self.n_kv_heads, max_keys, ctx.runtime.sm_count)
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(kernels.split_scratch_floats(T, self.n_heads, self.head_dim, n_splits),
                                      dtype=torch.float32, device=dev)
            kernels.attention(q, out, k_pages=kv.k_pages, v_pages=kv.v_pages, block_table=kv.block_table,
                              table_width=kv.table_width, ring_pages=kv.ring_pages, page_tokens=kv.page_tokens,
                              n_splits=n_splits, scratch=scratch, **common)
        kernels.mark("attention")
        kernels.linear(out, self.w_o, bias=self.b_o, out=residual, accumulate=True)
        kernels.mark("o")
