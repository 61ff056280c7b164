"""Other kinds of parts, defined here and plugged in without touching the
package: a feed-forward with routing (top-1 of several small experts, router
logits in float32) and another position encoding (a learned vector per
position added to q and k instead of a rotation).  One toy architecture uses
the new position encoding in its first layer and the routed feed-forward in
its second; the engine steps it whole, in unequal batches and token by token,
and a plain computation written here follows (GPU).  The toys' own arithmetic
uses torch operations and the package's kernels as building blocks: they are
test doubles, not models of anyone's.
"""
import math

import pytest
import torch

import plain_model as pm
from helpers import TINY_A, assert_close, random_tokens

pytestmark = pytest.mark.gpu
N_EXPERTS, EXPERT_WIDTH, MAX_POS = 3, 40, 512


def _register():
    from dataclasses import replace

    from tq_kv_b200 import kernels
    from tq_kv_b200.config import Architecture, PartSpec, Qwen2Config, build_qwen2_spec, register_architecture
    from tq_kv_b200.parts import FeedForward, PositionEncoding, WeightSpec, register_part

    class RoutedFeedForward(FeedForward):
        """Top-1 routing over small SwiGLU experts; the router runs in float32."""
        graph_capturable = False          # which rows go to which expert is decided on the host

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.n, self.width = (self.params[k] for k in ("hidden_size", "experts", "expert_width"))

        def weight_specs(self):
            p = self.prefix
            specs = [WeightSpec(p + "router.weight", (self.n, self.hidden), "matrix")]
            for e in range(self.n):
                specs += [WeightSpec(f"{p}experts.{e}.gate_up.weight", (2 * self.width, self.hidden), "matrix"),
                          WeightSpec(f"{p}experts.{e}.down.weight", (self.hidden, self.width), "matrix")]
            return specs

        def bind(self, tensors, runtime, shared=None):
            p = self.prefix
            self.router = tensors[p + "router.weight"].float()
            self.gate_up = [tensors[f"{p}experts.{e}.gate_up.weight"].contiguous() for e in range(self.n)]
            self.down = [tensors[f"{p}experts.{e}.down.weight"].contiguous() for e in range(self.n)]

        def forward(self, x, ctx, residual):
            choice = (x.float() @ self.router.T).argmax(-1)
            for e in range(self.n):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel() == 0:
                    continue
                act = kernels.linear(x[rows].contiguous(), self.gate_up[e], swiglu=True, out_dtype=x.dtype)
                residual[rows] += kernels.linear(act, self.down[e], out_dtype=torch.float32)

    class LearnedPositions(PositionEncoding):
        """q and k get a learned vector of their position added; nothing is rotated.  The package's fused
        bias + rotation + cache-append kernel does the head split and the append, with tables of a zero angle."""

        def __init__(self, spec):
            super().__init__(spec)
            self.head_dim, self.max_pos = self.params["head_dim"], self.params["max_positions"]

        def weight_specs(self):
            return [WeightSpec(self.prefix + "table.weight", (self.max_pos, self.head_dim), "embedding")]

        def bind(self, tensors, runtime, shared=None):
            self.table = tensors[self.prefix + "table.weight"].float()

        def prepare(self, runtime, shared=None):
            self.cos = torch.ones(runtime.max_context, self.head_dim // 2, device=runtime.device)
            self.sin = torch.zeros_like(self.cos)

        def encode_and_store(self, qkv, bias, ctx, *, n_heads, n_kv_heads, head_dim, q_out, k_out, v_out):
            b, kv = ctx.batch, ctx.kv
            add = self.table[b.tok_pos.long()]                               # [T, head_dim]
            qk = qkv[:, :(n_heads + n_kv_heads) * head_dim].view(-1, n_heads + n_kv_heads, head_dim)
            if bias is not None:                                             # the bias comes before the encoding
                qkv += bias
            qk += add.unsqueeze(1)
            kernels.qkv_rope_cache(qkv, None, self.cos, self.sin, b.tok_pos, b.tok_seq, b.new_lens, q_out,
                                   n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, rotary_dim=head_dim,
                                   k_out=k_out, v_out=v_out, k_pages=kv.k_pages, v_pages=kv.v_pages,
                                   block_table=kv.block_table, table_width=kv.table_width,
                                   ring_pages=kv.ring_pages, page_tokens=kv.page_tokens)

    register_part("toy_routed_ffn", RoutedFeedForward, replace=True)
    register_part("toy_learned_positions", LearnedPositions, replace=True)

    def build(cfg):
        spec = build_qwen2_spec(cfg)
        l0, l1 = spec.layers
        mixer0 = replace(l0.mixer, params={**l0.mixer.params, "position": PartSpec(
            "toy_learned_positions", {"head_dim": cfg.head_dim, "max_positions": MAX_POS},
            "model.layers.0.self_attn.positions.")})
        ffn1 = PartSpec("toy_routed_ffn", {"hidden_size": cfg.hidden_size, "experts": N_EXPERTS,
                                           "expert_width": EXPERT_WIDTH}, "model.layers.1.moe.")
        return replace(spec, architecture="ToyPartsForCausalLM",
                       layers=(replace(l0, mixer=mixer0), replace(l1, feed_forward=ffn1)))

    register_architecture(Architecture("ToyPartsForCausalLM", "toyparts", Qwen2Config, build), replace=True)


def _plain(cfg, w, toks):
    T = len(toks)
    nh, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    cos, sin = pm.rope_tables(hd, cfg["rope_theta"], T)
    h = w["model.embed_tokens.weight"][torch.tensor(toks)]
    for i in range(2):
        p = f"model.layers.{i}."
        a = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = (a @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]).reshape(T, nh, hd)
        k = (a @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]).reshape(T, nkv, hd)
        v = (a @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]).reshape(T, nkv, hd)
        if i == 0:
            add = w[p + "self_attn.positions.table.weight"][:T].unsqueeze(1)
            q, k = (q + add).transpose(0, 1), (k + add).transpose(0, 1)
        else:
            q, k = pm.rope_halved(q.transpose(0, 1), cos, sin), pm.rope_halved(k.transpose(0, 1), cos, sin)
        k, v = pm.repeat_kv(k, nh // nkv), pm.repeat_kv(v.transpose(0, 1), nh // nkv)
        att = q @ k.transpose(1, 2) / math.sqrt(hd)
        att = torch.where(pm.attention_mask(T, None), torch.full_like(att, float("-inf")), att)
        y = (pm.softmax_last_dim(att) @ v).transpose(0, 1).reshape(T, nh * hd)
        h = h + y @ w[p + "self_attn.o_proj.weight"].T
        m = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        if i == 1:
            choice = (m @ w[p + "moe.router.weight"].T).argmax(-1)
            out = torch.zeros_like(h)
            for e in range(N_EXPERTS):
                rows = choice == e
                gu = m[rows] @ w[f"{p}moe.experts.{e}.gate_up.weight"].T
                out[rows] = (torch.nn.functional.silu(gu[:, :EXPERT_WIDTH]) * gu[:, EXPERT_WIDTH:]) @ \
                    w[f"{p}moe.experts.{e}.down.weight"].T
            h = h + out
        else:
            h = h + pm.swiglu_mlp(m, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                  w[p + "mlp.down_proj.weight"])
    return pm.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    from tq_kv_b200.config import unregister_architecture
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.parts import unregister_part
    from tq_kv_b200.weights import write_model_folder
    _register()
    try:
        cfg = {**TINY_A, "architectures": ["ToyPartsForCausalLM"]}
        folder = write_model_folder(cfg, str(tmp_path / "toyparts"), seed=6)
        c, w = pm.read_model_folder(folder)
        assert "model.layers.1.moe.router.weight" in w and "model.layers.0.self_attn.positions.table.weight" in w
        assert "model.layers.1.mlp.gate_proj.weight" not in w
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=3)
        reqs = [random_tokens(n, 256, 80 + n) for n in (70, 33, 12)]
        wants = [_plain(c, w, t) for t in reqs]
        for toks, want in zip(reqs, wants):
            s = eng.new_sequence()
            assert_close(eng.step([StepRow(s, toks, list(range(len(toks))))]), want, "float32", "whole")
            eng.release(s)
        slots = [eng.new_sequence() for _ in reqs]
        cut = [40, 30, 1]
        got = eng.step([StepRow(s, t[:n], [n - 1]) for s, t, n in zip(slots, reqs, cut)])
        assert_close(got, torch.stack([w_[n - 1] for w_, n in zip(wants, cut)]), "float32", "prompts")
        live = [0, 1, 2]
        while live:
            got = eng.step([StepRow(slots[i], [reqs[i][cut[i]]], [0]) for i in live])
            assert_close(got, torch.stack([wants[i][cut[i]] for i in live]), "float32", "decode")
            for i in list(live):
                cut[i] += 1
                if cut[i] == len(reqs[i]):
                    eng.release(slots[i])
                    live.remove(i)
    finally:
        unregister_architecture("ToyPartsForCausalLM")
        unregister_part("toy_routed_ffn")
        unregister_part("toy_learned_positions")
