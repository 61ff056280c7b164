"""A mixer with state of its own, defined here, is registered, built into an
architecture, given state by the cache and stepped — without a change to the
package's files (GPU).

The toy mixer keeps, per sequence, the running sum of its (projected) inputs:
    s_t = s_{t-1} + x_t W_in^T ;  y_t = (s_t / (t + 1)) W_out^T
Its state has a fixed size per sequence whatever the sequence's length.  A
layer with this mixer sits between two attention layers, so that one model
mixes mixers.  (The toy's own arithmetic uses torch operations: it is a test
double, not a product kernel.)
"""
import pytest
import torch

import plain_model as pm
from helpers import TINY_A, assert_close, random_tokens

pytestmark = pytest.mark.gpu


def _register(capturable=False):
    from dataclasses import replace

    from tq_kv_b200.cache import StateRequest
    from tq_kv_b200.config import (Architecture, LayerSpec, PartSpec, Qwen2Config, ScheduleEntry, build_qwen2_spec,
                                   register_architecture)
    from tq_kv_b200.parts import Mixer, WeightSpec, register_part

    class RunningMeanMixer(Mixer):
        graph_capturable = capturable     # False: every step reads the batch's layout back to the host

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.inner = self.params["hidden_size"], self.params["inner_size"]

        def weight_specs(self):
            return [WeightSpec(self.prefix + "in.weight", (self.inner, self.hidden), "matrix"),
                    WeightSpec(self.prefix + "out.weight", (self.hidden, self.inner), "matrix")]

        def bind(self, tensors, runtime, shared=None):
            self.w_in = tensors[self.prefix + "in.weight"].float()
            self.w_out = tensors[self.prefix + "out.weight"].float()

        def state_request(self):
            return StateRequest((self.inner,), torch.float32)

        def forward(self, x, ctx, residual):
            b = ctx.batch
            u = x.float() @ self.w_in.T
            if capturable and b.single_tokens:
                # one token per row: everything stays on the device, so the step can be captured and replayed
                slots = b.slots.long()
                ctx.state.index_add_(0, slots, u)
                residual += (ctx.state[slots] / (b.tok_pos + 1).unsqueeze(1)) @ self.w_out.T
                return
            cu = b.cu_seqlens.tolist()
            for row, slot in enumerate(b.host_slots):
                a, e = cu[row], cu[row + 1]
                s = ctx.state[slot] + torch.cumsum(u[a:e], 0)
                n = torch.arange(b.host_start[row] + 1, b.host_start[row] + e - a + 1, device=x.device)
                residual[a:e] += (s / n.unsqueeze(1)) @ self.w_out.T
                ctx.state[slot] = s[-1]

    register_part("toy_running_mean", RunningMeanMixer, replace=True)

    def build(cfg):
        spec = build_qwen2_spec(cfg)
        mid = spec.layers[1]
        toy = replace(mid, mixer=PartSpec("toy_running_mean", {"hidden_size": cfg.hidden_size, "inner_size": 24},
                                          "model.layers.1.toy."))
        return replace(spec, architecture="ToyMixForCausalLM", layers=(spec.layers[0], toy, spec.layers[2]))

    register_architecture(Architecture("ToyMixForCausalLM", "toymix", Qwen2Config, build), replace=True)


def _plain(cfg, w, toks):
    """The same model from the plain implementation's parts."""
    T = len(toks)
    eps, hd = cfg["rms_norm_eps"], cfg["head_dim"]
    cos, sin = pm.rope_tables(hd, cfg["rope_theta"], T)
    h = w["model.embed_tokens.weight"][torch.tensor(toks)]
    for i in range(3):
        p = f"model.layers.{i}."
        a = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if i == 1:
            u = torch.cumsum(a @ w[p + "toy.in.weight"].T, 0) / torch.arange(1, T + 1).unsqueeze(1)
            h = h + u @ w[p + "toy.out.weight"].T
        else:
            h = h + pm.attention(a, *[w[f"{p}self_attn.{n}_proj.{l}"] for n in "qkv" for l in ("weight", "bias")],
                                 w[p + "self_attn.o_proj.weight"], cfg["num_attention_heads"],
                                 cfg["num_key_value_heads"], hd, cos, sin, None)
        m = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + pm.swiglu_mlp(m, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                              w[p + "mlp.down_proj.weight"])
    return pm.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from tq_kv_b200.config import unregister_architecture
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.parts import unregister_part
    from tq_kv_b200.weights import write_model_folder
    _register()
    try:
        cfg = {**TINY_A, "architectures": ["ToyMixForCausalLM"], "num_hidden_layers": 3, "max_window_layers": 3}
        folder = write_model_folder(cfg, str(tmp_path / "toy"), seed=4)
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=3)
        assert list(eng.cache.state) == [1] and tuple(eng.cache.state[1].shape) == (3, 24)
        assert sorted(eng.cache.group_of_entry) == [0, 2]           # the toy layer asks for no keys or values
        c, w = pm.read_model_folder(folder)
        reqs = [random_tokens(n, 256, 40 + n) for n in (50, 21, 9)]
        wants = [_plain(c, w, t) for t in reqs]
        # whole
        for toks, want in zip(reqs, wants):
            s = eng.new_sequence()
            assert_close(eng.step([StepRow(s, toks, list(range(len(toks))))]), want, "float32", "whole")
            eng.release(s)
        # an unequal batch, prompts then one token each; a slot is reused in between
        slots = [eng.new_sequence() for _ in reqs]
        cut = [30, 20, 1]
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
        s = eng.new_sequence()                                      # reused slot: its state starts from zero again
        assert_close(eng.step([StepRow(s, reqs[2], [8])]), wants[2][8:9], "float32", "reused slot")
        eng.release(s)
    finally:
        unregister_architecture("ToyMixForCausalLM")
        unregister_part("toy_running_mean")


def test_a_stateful_mixer_in_replayed_graphs_advances_its_state_once_per_step(tmp_path):
    """Decode steps of a model whose mixer keeps state are captured and
    replayed; the first step of every batch size runs once, not twice, so the
    logits equal those of plain launches and of the plain implementation."""
    from tq_kv_b200.config import unregister_architecture
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.parts import unregister_part
    from tq_kv_b200.weights import write_model_folder
    _register(capturable=True)
    try:
        cfg = {**TINY_A, "architectures": ["ToyMixForCausalLM"], "num_hidden_layers": 3, "max_window_layers": 3}
        folder = write_model_folder(cfg, str(tmp_path / "toy"), seed=5)
        c, w = pm.read_model_folder(folder)
        reqs = [random_tokens(n, 256, 70 + n) for n in (30, 12, 20)]
        wants = [_plain(c, w, t) for t in reqs]
        outs = {}
        for graphs in (True, False):
            eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=3)
            assert eng.use_graphs                       # the toy part declares itself capturable
            assert not eng.pad_prompts                  # but not that padded rows are harmless (it keeps state)
            eng.use_graphs = graphs
            slots = [eng.new_sequence() for _ in reqs]
            cut = [6, 4, 5]
            eng.step([StepRow(s, t[:c_], []) for s, t, c_ in zip(slots, reqs, cut)])
            got, live = [], [0, 1, 2]
            while live:                                 # batch sizes 3, 2, 1: three first uses of a graph
                out = eng.step([StepRow(slots[i], [reqs[i][cut[i]]], [0]) for i in live])
                assert_close(out, torch.stack([wants[i][cut[i]] for i in live]), "float32",
                             f"graphs={graphs}, decode at {[cut[i] for i in live]}")
                got.append(out.clone())
                for i in list(live):
                    cut[i] += 1
                    if cut[i] == len(reqs[i]):
                        eng.release(slots[i])
                        live.remove(i)
            outs[graphs] = torch.cat(got)
            if graphs:
                assert sorted(eng._decode_graphs) == [1, 2, 3]
        # the two differ by rounding only: a graph plans attention's splits for the context limit
        assert_close(outs[True], outs[False].cpu(), "float32", "graph vs plain launches")
    finally:
        unregister_architecture("ToyMixForCausalLM")
        unregister_part("toy_running_mean")
