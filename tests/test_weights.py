"""Weights: file format, loading by name with one collected error, dtype
policy, the random-weights mode (CPU)."""
import json
import os

import pytest
import torch

import plain_model
from helpers import TINY_A, TINY_B
from tq_kv_b200.config import spec_from_config_dict
from tq_kv_b200.engine import DecoderModel
from tq_kv_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_tensors, target_dtype,
                                write_model_folder, write_safetensors)


def _expected(cfg):
    _, _, spec = spec_from_config_dict(cfg)
    m = DecoderModel(spec)
    return {n: tuple(ws.shape) for n, ws in m.weight_specs().items()}, m.ignored_weights()


def test_write_then_read_round_trip(tmp_path):
    a = torch.randn(3, 5)
    b = torch.randn(7).to(torch.bfloat16)
    c = torch.arange(6, dtype=torch.int64).reshape(2, 3)
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, [("a", a.dtype, tuple(a.shape)), ("b", b.dtype, tuple(b.shape)), ("c", c.dtype, (2, 3))],
                      [("a", a), ("b", b), ("c", c)])
    f = SafetensorsFile(p)
    assert torch.equal(f.read("a"), a) and torch.equal(f.read("b"), b) and torch.equal(f.read("c"), c)
    f.close()
    # an independent reader agrees
    os.rename(p, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text("{}")
    _, t = plain_model.read_model_folder(str(tmp_path))
    assert torch.equal(t["a"], a) and torch.equal(t["b"], b.float())


def test_random_folder_has_exactly_the_expected_tensors(tmp_path):
    for name, cfg in (("a", TINY_A), ("b", TINY_B)):
        folder = write_model_folder(cfg, str(tmp_path / name), seed=3)
        expected, ignored = _expected(cfg)
        got = load_tensors(folder, expected, ignored, mode=torch.float32, device="cpu")
        assert set(got) == set(expected)
        assert all(tuple(got[n].shape) == expected[n] for n in expected)
        assert ("lm_head.weight" in expected) == (not cfg["tie_word_embeddings"])
        norm = got["model.norm.weight"]
        assert abs(float(norm.mean()) - 1.0) < 0.1 and 0.03 < float(got["model.embed_tokens.weight"].std()) * 2 < 0.05
        assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["Qwen2ForCausalLM"]


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    f1 = write_model_folder(TINY_A, str(tmp_path / "s1"), seed=5)
    f2 = write_model_folder(TINY_A, str(tmp_path / "s2"), seed=5)
    f3 = write_model_folder(TINY_A, str(tmp_path / "s3"), seed=6)
    _, w1 = plain_model.read_model_folder(f1)
    _, w2 = plain_model.read_model_folder(f2)
    _, w3 = plain_model.read_model_folder(f3)
    assert all(torch.equal(w1[k], w2[k]) for k in w1)
    assert not torch.equal(w1["model.embed_tokens.weight"], w3["model.embed_tokens.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_model_folder(TINY_B, str(tmp_path / "m"), seed=1)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.read(n).clone() for n in f.entries}
    f.close()
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(2)
    tensors["model.layers.2.mlp.up_proj.weight"] = torch.zeros(200, 95)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()], list(tensors.items()))
    expected, ignored = _expected(TINY_B)
    with pytest.raises(WeightsError) as ei:
        load_tensors(folder, expected, ignored, mode=torch.bfloat16, device="cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert e.wrong_shape == [("model.layers.2.mlp.up_proj.weight", (200, 95), (200, 96))]
    msg = str(e)
    for needle in ("missing tensors (2)", "k_proj.bias", "unexpected tensors (1)", "extra.weight", "wrong shapes (1)",
                   "[200, 95]", "[200, 96]"):
        assert needle in msg


def test_tied_model_may_carry_an_unused_head(tmp_path):
    folder = write_model_folder(TINY_A, str(tmp_path / "m"), seed=1)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.read(n).clone() for n in f.entries}
    f.close()
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()], list(tensors.items()))
    expected, ignored = _expected(TINY_A)
    assert "lm_head.weight" in ignored
    assert "lm_head.weight" not in load_tensors(folder, expected, ignored, mode=torch.float32, device="cpu")


def test_dtype_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(torch.bfloat16, bf) == bf and target_dtype(torch.float16, bf) == bf
    assert target_dtype(torch.float32, bf) == f32            # a tensor stored in 32-bit stays so
    assert target_dtype(torch.int64, bf) == torch.int32 and target_dtype(torch.int64, f32) == torch.int32
    assert target_dtype(torch.bfloat16, f32) == f32


def test_mixed_storage_is_kept_per_tensor(tmp_path):
    p = str(tmp_path / "model.safetensors")
    a, b, c = torch.randn(4, 4).to(torch.bfloat16), torch.randn(4), torch.arange(4)
    write_safetensors(p, [("a", a.dtype, (4, 4)), ("b", b.dtype, (4,)), ("c", c.dtype, (4,))],
                      [("a", a), ("b", b), ("c", c)])
    got = load_tensors(str(tmp_path), {"a": (4, 4), "b": (4,), "c": (4,)}, [], mode=torch.bfloat16, device="cpu")
    assert got["a"].dtype == torch.bfloat16 and got["b"].dtype == torch.float32 and got["c"].dtype == torch.int32
    assert torch.equal(got["b"], b)


def test_file_errors(tmp_path):
    with pytest.raises(SafetensorsError, match="No .safetensors files"):
        load_tensors(str(tmp_path), {}, [], mode=torch.float32, device="cpu")
    (tmp_path / "bad.safetensors").write_bytes(b"\xff" * 4)
    with pytest.raises(SafetensorsError):
        load_tensors(str(tmp_path), {}, [], mode=torch.float32, device="cpu")


def test_random_weights_depend_on_seed_name_and_element_only():
    from tq_kv_b200.weights.random_init import random_tensor, standard_normal_host, tensor_key
    a = random_tensor("x.weight", (7, 9), "matrix", 3, torch.float32, "cpu")
    assert torch.equal(a, random_tensor("x.weight", (7, 9), "matrix", 3, torch.float32, "cpu"))
    assert torch.equal(a.flatten()[:20], random_tensor("x.weight", (20,), "matrix", 3, torch.float32, "cpu"))
    assert not torch.equal(a, random_tensor("y.weight", (7, 9), "matrix", 3, torch.float32, "cpu"))
    assert not torch.equal(a, random_tensor("x.weight", (7, 9), "matrix", 4, torch.float32, "cpu"))
    key = tensor_key(3, "x.weight")
    whole = standard_normal_host(key, 0, 5000)
    assert (standard_normal_host(key, 1234, 100) == whole[1234:1334]).all()       # any range, any chunking
    b = random_tensor("x.weight", (7, 9), "matrix", 3, torch.bfloat16, "cpu")
    assert torch.equal(b, a.to(torch.bfloat16))                                    # rounded once, from float32


def test_random_weights_are_normal_with_the_roles_moments():
    from tq_kv_b200.weights.random_init import random_tensor
    m = random_tensor("m", (400, 500), "matrix", 1, torch.float32, "cpu").double()
    assert abs(float(m.mean())) < 2e-4 and abs(float(m.std()) - 0.02) < 2e-4
    z = m / 0.02
    assert abs(float((z ** 3).mean())) < 0.03 and abs(float((z ** 4).mean()) - 3.0) < 0.06
    assert float(z.abs().max()) < 5.8 and torch.isfinite(m).all()
    n = random_tensor("n", (4096,), "norm_scale", 1, torch.float32, "cpu").double()
    assert abs(float(n.mean()) - 1.0) < 6e-3 and abs(float(n.std()) - 0.1) < 6e-3


def _split_into_shards(folder, tmp_path, name="sharded"):
    """The folder's tensors in two shard files (odd and even tensors) under a new folder."""
    import shutil
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.read(n).clone() for n in f.entries}
    f.close()
    out = str(tmp_path / name)
    os.makedirs(out)
    shutil.copy(os.path.join(folder, "config.json"), out)
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[0::2], "model-00002-of-00002.safetensors": names[1::2]}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(out, fname), [(n, tensors[n].dtype, tuple(tensors[n].shape)) for n in ns],
                          [(n, tensors[n]) for n in ns])
    return out, parts, tensors


def test_shards_are_found_by_scan_and_by_the_index(tmp_path):
    from tq_kv_b200.weights.safetensors_io import INDEX_NAME
    folder = write_model_folder(TINY_A, str(tmp_path / "whole"), seed=2)
    expected, ignored = _expected(TINY_A)
    whole = load_tensors(folder, expected, ignored, mode=torch.float32, device="cpu")
    out, parts, tensors = _split_into_shards(folder, tmp_path)
    scanned = load_tensors(out, expected, ignored, mode=torch.float32, device="cpu")      # no index: the folder scan
    assert all(torch.equal(whole[n], scanned[n]) for n in whole)
    # a tensor stored in two shards is an error of the scan ...
    dup = sorted(tensors)[0]
    write_safetensors(os.path.join(out, "stray.safetensors"), [(dup, tensors[dup].dtype, tuple(tensors[dup].shape))],
                      [(dup, torch.zeros_like(tensors[dup]))])
    with pytest.raises(SafetensorsError, match="stored twice"):
        load_tensors(out, expected, ignored, mode=torch.float32, device="cpu")
    # ... but with an index the weight_map decides, and the stray file is not read
    weight_map = {n: fname for fname, ns in parts.items() for n in ns}
    with open(os.path.join(out, INDEX_NAME), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    indexed = load_tensors(out, expected, ignored, mode=torch.float32, device="cpu")
    assert all(torch.equal(whole[n], indexed[n]) for n in whole)
    # an index that places a tensor in the wrong file, or names a file that is not there, is an error
    bad = dict(weight_map)
    bad[dup] = [f for f in parts if f != weight_map[dup]][0]
    with open(os.path.join(out, INDEX_NAME), "w") as f:
        json.dump({"weight_map": bad}, f)
    with pytest.raises(SafetensorsError, match="do not hold them"):
        load_tensors(out, expected, ignored, mode=torch.float32, device="cpu")
    bad = dict(weight_map)
    bad[dup] = "model-00003-of-00002.safetensors"
    with open(os.path.join(out, INDEX_NAME), "w") as f:
        json.dump({"weight_map": bad}, f)
    with pytest.raises(SafetensorsError, match="not in"):
        load_tensors(out, expected, ignored, mode=torch.float32, device="cpu")
    with open(os.path.join(out, INDEX_NAME), "w") as f:
        f.write("{")
    with pytest.raises(SafetensorsError, match="Invalid model.safetensors.index.json"):
        load_tensors(out, expected, ignored, mode=torch.float32, device="cpu")
