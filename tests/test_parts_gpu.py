"""Each part alone: built from a PartSpec, bound to random tensors, run on a
small step, compared with the plain implementation's function for that part
(GPU).  Sizes differ from both tiny models."""
import math

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _runtime(dtype=torch.float32, max_context=256):
    from tq_kv_b200.parts import Runtime
    return Runtime(device=torch.device(DEV), act_dtype=dtype, max_context=max_context)


def _bind_random(part, runtime, seed=0):
    from tq_kv_b200.weights import random_tensors
    specs = list(part.weight_specs())
    pos = getattr(part, "position", None)
    if pos is not None:
        specs += pos.weight_specs()
    tensors = dict(random_tensors(specs, seed, torch.float32, DEV))
    part.bind(tensors, runtime, {})
    return {k: v.cpu() for k, v in tensors.items()}


def _step(cache, rows):
    """Reserves, packs and commits a step for a part-level test."""
    from tq_kv_b200.engine import build_step_batch
    slots, lens = [r.slot for r in rows], [len(r.tokens) for r in rows]
    cache.reserve(slots, lens)
    batch = build_step_batch(rows, cache, DEV)
    return batch, lambda: cache.commit(slots, lens)


def test_rms_norm_part():
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.parts import make_part
    part = make_part(PartSpec("rms_norm", {"width": 120, "eps": 3e-4}, "n."))
    w = _bind_random(part, _runtime())
    x = torch.randn(9, 120, device=DEV) * 2
    got = part.forward(x, torch.float32)
    assert torch.allclose(got.cpu(), pm.rms_norm(x.cpu(), w["n.weight"], 3e-4), atol=1e-6)
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    assert torch.equal(part.forward(x, torch.float32, rows), got[[8, 2]])


def test_rotary_tables_equal_the_plain_tables():
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.parts import make_part
    part = make_part(PartSpec("rotary_halved", {"head_dim": 48, "rotary_dim": 48, "theta": 1e6}))
    part.prepare(_runtime(max_context=300))
    cos, sin = pm.rope_tables(48, 1e6, 300)
    assert torch.equal(part.cos.cpu(), cos) and torch.equal(part.sin.cpu(), sin)


def test_embedding_and_head_parts():
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.parts import make_part
    rt = _runtime()
    emb = make_part(PartSpec("token_embedding", {"vocab_size": 333, "width": 40}, "e."))
    w = _bind_random(emb, rt)
    toks = torch.tensor([0, 332, 7], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(toks).cpu(), w["e.weight"][toks.long().cpu()])
    head = make_part(PartSpec("lm_head", {"vocab_size": 333, "width": 40, "tied_to": "e.weight"}, "h."))
    assert [s.name for s in head.weight_specs()] == ["e.weight"] and head.ignored_weights() == ["h.weight"]
    head.bind({"e.weight": emb.table}, rt, {})
    x = torch.randn(5, 40, device=DEV)
    assert torch.allclose(head.forward(x).cpu(), x.cpu() @ w["e.weight"].T, atol=1e-5)
    own = make_part(PartSpec("lm_head", {"vocab_size": 333, "width": 40, "tied_to": None}, "h."))
    assert [s.name for s in own.weight_specs()] == ["h.weight"]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_swiglu_part(dtype, tol):
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.parts import StepContext, make_part
    rt = _runtime(dtype)
    part = make_part(PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 150}, "mlp."))
    w = _bind_random(part, rt)
    for T in (3, 40):                                   # the few-rows kernel and the many-rows kernel
        x = torch.randn(T, 72, device=DEV)
        res = torch.randn(T, 72, device=DEV)
        want = res.cpu() + pm.swiglu_mlp(x.to(dtype).float().cpu(), w["mlp.gate_proj.weight"],
                                         w["mlp.up_proj.weight"], w["mlp.down_proj.weight"])
        part.forward(x.to(dtype), StepContext(batch=None, runtime=rt, entry=0), res)
        assert float((res.cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("window", [None, 24])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_attention_part_prompt_then_decode(window, dtype, tol):
    """The mixer alone with a cache of its own: a prompt of 50, then 30 single
    tokens, two sequences of different length side by side."""
    from tq_kv_b200.cache import KVLayerView, SequenceCache
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.engine import StepRow
    from tq_kv_b200.parts import StepContext, make_part
    H, nh, nkv, hd = 56, 6, 2, 48
    rt = _runtime(dtype)
    part = make_part(PartSpec("gqa_attention", {
        "hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": True, "window": window,
        "position": PartSpec("rotary_halved", {"head_dim": hd, "rotary_dim": hd, "theta": 5e4})}, "a."))
    w = _bind_random(part, rt)
    cache = SequenceCache({0: part.cache_request()}, {}, max_tokens=512, max_slots=2, max_length=256, dtype=dtype,
                          device=DEV)
    lens = [80, 61]
    xs = [torch.randn(n, H) for n in lens]
    cos, sin = pm.rope_tables(hd, 5e4, 256)
    wants = [pm.attention(x.to(dtype).float(), w["a.q_proj.weight"], w["a.q_proj.bias"], w["a.k_proj.weight"],
                          w["a.k_proj.bias"], w["a.v_proj.weight"], w["a.v_proj.bias"], w["a.o_proj.weight"],
                          nh, nkv, hd, cos, sin, window) for x in xs]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    at = [0, 0]

    def run(chunks):
        rows = [StepRow(slots[i], [0] * n, []) for i, n in enumerate(chunks) if n]
        live = [i for i, n in enumerate(chunks) if n]
        batch, commit = _step(cache, rows)
        x = torch.cat([xs[i][at[i]:at[i] + chunks[i]] for i in live]).to(DEV)
        res = torch.zeros(x.shape[0], H, device=DEV)
        gi, kp, vp = cache.layer_pages(0)
        table, width = batch.block_tables[gi]
        g = cache.groups[gi]
        ctx = StepContext(batch=batch, runtime=rt, entry=0,
                          kv=KVLayerView(kp, vp, table, width, g.ring_pages, g.book.page_tokens, True))
        part.forward(x.to(dtype), ctx, res)
        commit()
        o = 0
        for i in live:
            want = wants[i][at[i]:at[i] + chunks[i]]
            got = res[o:o + chunks[i]].cpu()
            assert float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), (i, at[i])
            o += chunks[i]
            at[i] += chunks[i]

    run([50, 31])
    for _ in range(30):
        run([1, 1])
    assert at == lens


def test_prenorm_block():
    from tq_kv_b200.cache import KVLayerView, SequenceCache
    from tq_kv_b200.config import LayerSpec, PartSpec
    from tq_kv_b200.engine import StepRow
    from tq_kv_b200.parts import StepContext, make_block
    from tq_kv_b200.weights import random_tensors
    H, nh, nkv, hd, I = 40, 5, 1, 16, 90
    spec = LayerSpec(
        block="prenorm_residual",
        mixer=PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
                                         "qkv_bias": True, "window": None,
                                         "position": PartSpec("rotary_halved", {"head_dim": hd, "rotary_dim": hd,
                                                                                "theta": 1e4})}, "L.self_attn."),
        feed_forward=PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}, "L.mlp."),
        mixer_norm=PartSpec("rms_norm", {"width": H, "eps": 1e-6}, "L.input_layernorm."),
        feed_forward_norm=PartSpec("rms_norm", {"width": H, "eps": 1e-6}, "L.post_attention_layernorm."))
    block = make_block(spec)
    rt = _runtime()
    specs = [ws for p in block.parts() for ws in p.weight_specs()]
    tensors = dict(random_tensors(specs, 1, torch.float32, DEV))
    for p in block.parts():
        p.bind(tensors, rt, {})
    w = {k: v.cpu() for k, v in tensors.items()}
    cache = SequenceCache({0: block.mixer.cache_request()}, {}, max_tokens=128, max_slots=1, max_length=128,
                          dtype=torch.float32, device=DEV)
    T = 21
    h0 = torch.randn(T, H)
    cos, sin = pm.rope_tables(hd, 1e4, T)
    a = pm.rms_norm(h0, w["L.input_layernorm.weight"], 1e-6)
    h1 = h0 + pm.attention(a, *[w[f"L.self_attn.{n}_proj.{leaf}"] for n in "qkv" for leaf in ("weight", "bias")],
                           w["L.self_attn.o_proj.weight"], nh, nkv, hd, cos, sin, None)
    m = pm.rms_norm(h1, w["L.post_attention_layernorm.weight"], 1e-6)
    want = h1 + pm.swiglu_mlp(m, w["L.mlp.gate_proj.weight"], w["L.mlp.up_proj.weight"], w["L.mlp.down_proj.weight"])
    s = cache.alloc_slot()
    batch, commit = _step(cache, [StepRow(s, [0] * T, [])])
    gi, kp, vp = cache.layer_pages(0)
    table, width = batch.block_tables[gi]
    h = h0.to(DEV)
    block.forward(h, StepContext(batch=batch, runtime=rt, entry=0,
                                 kv=KVLayerView(kp, vp, table, width, 0, 64, True)))
    assert torch.allclose(h.cpu(), want, atol=3e-6)
