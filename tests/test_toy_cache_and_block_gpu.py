"""Two more toys plugged in from a test, without a change to the package:
a mixer whose cached key rows (24 wide) and value rows (8 wide) differ in
width, and a block kind with other slots than the package's own (a norm
after the mixer and after the feed-forward, named in `extra_parts`).  The
second layer of a toy architecture uses both; the engine steps it whole, in
an unequal batch and token by token, against a plain computation written here
(GPU).  The toys' arithmetic is torch operations: they are test doubles, not
models of anyone's.
"""
import math

import pytest
import torch

import plain_model as pm
from helpers import TINY_A, assert_close, random_tokens

pytestmark = pytest.mark.gpu
KEY_DIM, VALUE_DIM = 24, 8


def _register():
    from dataclasses import replace

    from tq_kv_b200.cache import KVRequest
    from tq_kv_b200.config import Architecture, PartSpec, Qwen2Config, build_qwen2_spec, register_architecture
    from tq_kv_b200.parts import Mixer, WeightSpec, make_part, register_block, register_part

    class NarrowValueAttention(Mixer):
        """One head, no position encoding: scores from 24-wide keys, outputs from 8-wide values."""
        graph_capturable = False          # walks the batch's rows on the host

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden = self.params["hidden_size"]

        def weight_specs(self):
            p = self.prefix
            return [WeightSpec(p + "q.weight", (KEY_DIM, self.hidden), "matrix"),
                    WeightSpec(p + "k.weight", (KEY_DIM, self.hidden), "matrix"),
                    WeightSpec(p + "v.weight", (VALUE_DIM, self.hidden), "matrix"),
                    WeightSpec(p + "o.weight", (self.hidden, VALUE_DIM), "matrix")]

        def bind(self, tensors, runtime, shared=None):
            self.w = {n: tensors[f"{self.prefix}{n}.weight"].float() for n in "qkvo"}

        def cache_request(self):
            return KVRequest(1, KEY_DIM, None, value_dim=VALUE_DIM)

        def forward(self, x, ctx, residual):
            b, kv = ctx.batch, ctx.kv
            assert kv.k_pages.shape[1:] == (1, kv.page_tokens, KEY_DIM)
            assert kv.v_pages.shape[1:] == (1, kv.page_tokens, VALUE_DIM)
            x = x.float()
            q, k, v = (x @ self.w[n].T for n in "qkv")
            cu = b.cu_seqlens.tolist()
            table = kv.block_table.reshape(-1, kv.table_width).tolist()
            for row in range(b.n_seqs):
                a, e, start = cu[row], cu[row + 1], b.host_start[row]
                for i in range(a, e):                       # append this row's keys and values to its pages
                    pos = start + i - a
                    page = table[row][pos // kv.page_tokens]
                    kv.k_pages[page, 0, pos % kv.page_tokens] = k[i].to(kv.k_pages.dtype)
                    kv.v_pages[page, 0, pos % kv.page_tokens] = v[i].to(kv.v_pages.dtype)
                n = start + e - a
                pages = torch.tensor(table[row][:-(-n // kv.page_tokens)], device=x.device)
                keys = kv.k_pages[pages, 0].reshape(-1, KEY_DIM)[:n].float()
                vals = kv.v_pages[pages, 0].reshape(-1, VALUE_DIM)[:n].float()
                s = q[a:e] @ keys.T / math.sqrt(KEY_DIM)
                j = torch.arange(n, device=x.device).unsqueeze(0)
                i = torch.arange(start, n, device=x.device).unsqueeze(1)
                s = s.masked_fill(j > i, float("-inf"))
                residual[a:e] += (torch.softmax(s, -1) @ vals) @ self.w["o"].T

    class SandwichBlock:
        """h += norm_after(mixer(norm_before(h))); the same around the feed-forward."""

        def __init__(self, spec):
            self.spec = spec
            self.names = ["mixer_norm", "mixer", "mixer_post_norm", "feed_forward_norm", "feed_forward",
                          "feed_forward_post_norm"]
            for n in self.names:
                setattr(self, n, make_part(spec.part(n)))

        def parts(self):
            return [getattr(self, n) for n in self.names]

        def forward(self, h, ctx):
            for pre, part, post in ((self.mixer_norm, self.mixer, self.mixer_post_norm),
                                    (self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm)):
                out = torch.zeros_like(h)
                part.forward(pre.forward(h, ctx.runtime.act_dtype), ctx, out)
                h += post.forward(out, torch.float32)

    register_part("toy_narrow_value_attention", NarrowValueAttention, replace=True)
    register_block("toy_sandwich", SandwichBlock, replace=True)

    def build(cfg):
        spec = build_qwen2_spec(cfg)
        one = spec.layers[1]
        norm = dict(one.mixer_norm.params)
        p = "model.layers.1."
        toy = replace(one, block="toy_sandwich",
                      mixer=PartSpec("toy_narrow_value_attention", {"hidden_size": cfg.hidden_size}, p + "toy."),
                      extra_parts={"mixer_post_norm": PartSpec("rms_norm", norm, p + "post_mixer_norm."),
                                   "feed_forward_post_norm": PartSpec("rms_norm", norm, p + "post_ffn_norm.")})
        return replace(spec, architecture="ToyCacheForCausalLM", layers=(spec.layers[0], toy))

    register_architecture(Architecture("ToyCacheForCausalLM", "toycache", Qwen2Config, build), replace=True)


def _plain(cfg, w, toks):
    T, eps, hd = len(toks), cfg["rms_norm_eps"], cfg["head_dim"]
    cos, sin = pm.rope_tables(hd, cfg["rope_theta"], T)
    h = w["model.embed_tokens.weight"][torch.tensor(toks)]
    p = "model.layers.0."
    a = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
    h = h + pm.attention(a, *[w[f"{p}self_attn.{n}_proj.{l}"] for n in "qkv" for l in ("weight", "bias")],
                         w[p + "self_attn.o_proj.weight"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                         hd, cos, sin, None)
    m = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    h = h + pm.swiglu_mlp(m, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    p = "model.layers.1."
    a = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
    q, k, v = (a @ w[f"{p}toy.{n}.weight"].T for n in "qkv")
    s = (q @ k.T / math.sqrt(KEY_DIM)).masked_fill(pm.attention_mask(T, None), float("-inf"))
    y = (pm.softmax_last_dim(s) @ v) @ w[p + "toy.o.weight"].T
    h = h + pm.rms_norm(y, w[p + "post_mixer_norm.weight"], eps)
    m = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    f = pm.swiglu_mlp(m, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    h = h + pm.rms_norm(f, w[p + "post_ffn_norm.weight"], eps)
    return pm.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


def test_unequal_key_and_value_widths_and_a_block_with_other_slots(tmp_path):
    from tq_kv_b200.config import ConfigError, unregister_architecture
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.parts import unregister_part
    from tq_kv_b200.weights import write_model_folder
    _register()
    try:
        cfg = {**TINY_A, "architectures": ["ToyCacheForCausalLM"]}
        folder = write_model_folder(cfg, str(tmp_path / "toy"), seed=6)
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=3)
        shapes = sorted((tuple(g.k.shape[2:]), tuple(g.v.shape[2:])) for g in eng.cache.groups)
        assert shapes == [((1, 64, KEY_DIM), (1, 64, VALUE_DIM)), ((2, 64, 16), (2, 64, 16))]
        c, w = pm.read_model_folder(folder)
        reqs = [random_tokens(n, 256, 90 + n) for n in (150, 70, 9)]
        wants = [_plain(c, w, t) for t in reqs]
        for toks, want in zip(reqs, wants):
            s = eng.new_sequence()
            assert_close(eng.step([StepRow(s, toks, list(range(len(toks))))]), want, "float32", "whole")
            eng.release(s)
        slots = [eng.new_sequence() for _ in reqs]
        cut = [130, 60, 1]
        got = eng.step([StepRow(s, t[:c_], [c_ - 1]) for s, t, c_ in zip(slots, reqs, cut)])
        assert_close(got, torch.stack([w_[c_ - 1] for w_, c_ in zip(wants, cut)]), "float32", "prompts")
        live = [0, 1, 2]
        while live:
            got = eng.step([StepRow(slots[i], [reqs[i][cut[i]]], [0]) for i in live])
            assert_close(got, torch.stack([wants[i][cut[i]] for i in live]), "float32", "decode")
            for i in list(live):
                cut[i] += 1
                if cut[i] == len(reqs[i]):
                    eng.release(slots[i])
                    live.remove(i)
        eng.cache.book.check()
        # a layer that lacks a slot its block kind needs is refused with the slot's name
        from dataclasses import replace

        from tq_kv_b200.config import Qwen2Config, build_qwen2_spec
        from tq_kv_b200.parts import make_block
        layer = build_qwen2_spec(Qwen2Config.from_dict(TINY_A)).layers[0]
        with pytest.raises(ConfigError, match="mixer_post_norm"):
            make_block(replace(layer, block="toy_sandwich"))
    finally:
        unregister_architecture("ToyCacheForCausalLM")
        unregister_part("toy_narrow_value_attention")
