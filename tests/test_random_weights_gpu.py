"""Random weights are the same on the host and on the device: the fill kernel
(csrc/random_fill.cu) and its numpy twin (weights/random_init.py) agree bit
for bit, so an engine filled on the GPU can be compared with the plain
implementation without a trip through a file (GPU)."""
import numpy as np
import pytest
import torch

import plain_model as pm
from helpers import TINY, assert_close, random_tokens, random_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("stored", ["float32", "bfloat16"])
def test_every_tensor_of_a_tiny_model_is_the_same_on_host_and_device(name, stored):
    cfg = {**TINY[name], "torch_dtype": stored}
    host = random_weights(cfg, 11, "cpu")
    dev = random_weights(cfg, 11, "cuda")
    assert sorted(host) == sorted(dev) and len(host) > 10
    for n, t in host.items():
        assert t.dtype == dev[n].dtype and torch.equal(t, dev[n].cpu()), n


def test_a_matrix_of_the_7b_shape_is_the_same_on_host_and_device():
    """18,944 x 3,584 values in bfloat16 from the kernel; the host twin is
    asked for ranges of the same stream: the start, the end, and places where
    the element index passes 2^24 and 2^26."""
    from tq_kv_b200.weights.random_init import random_tensor, standard_normal_host, tensor_key
    name, shape = "model.layers.3.mlp.gate_proj.weight", (18944, 3584)
    dev = random_tensor(name, shape, "matrix", 5, torch.bfloat16, "cuda").flatten()
    key = tensor_key(5, name)
    n = dev.numel()
    for start in (0, (1 << 24) - 5000, (1 << 26) - 5000, n - 100_000):
        want = torch.from_numpy(np.float32(0.0) + standard_normal_host(key, start, 100_000) * np.float32(0.02))
        assert torch.equal(dev[start:start + 100_000].cpu(), want.to(torch.bfloat16)), start
    f32 = random_tensor(name, (1 << 20,), "matrix", 5, torch.float32, "cuda")
    assert torch.equal(f32.cpu().to(torch.bfloat16), dev[:1 << 20].cpu())        # rounded once, from float32
    z = dev[:4_000_000].double() / 0.02
    assert abs(float(z.mean())) < 3e-3 and abs(float(z.std()) - 1.0) < 3e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_engine_with_random_weights_equals_the_plain_model_on_the_same_seed(dtype):
    from tq_kv_b200.engine import Engine, StepRow
    cfg = {**TINY["b"], "torch_dtype": "bfloat16"}
    eng = Engine.from_random(cfg, seed=21, dtype=dtype, max_tokens=256)
    toks = random_tokens(90, cfg["vocab_size"], 5)
    want = pm.decoder_logits(cfg, random_weights(cfg, 21, "cpu"), toks)
    s = eng.new_sequence()
    got = eng.step([StepRow(s, toks, list(range(len(toks))))])
    eng.release(s)
    assert_close(got, want, dtype, "from_random vs plain on host-made weights")


def test_a_folder_written_on_either_device_holds_the_same_bytes(tmp_path):
    from tq_kv_b200.weights import write_model_folder
    cfg = {**TINY["a"], "torch_dtype": "bfloat16"}
    a = write_model_folder(cfg, str(tmp_path / "host"), seed=3, device="cpu")
    b = write_model_folder(cfg, str(tmp_path / "device"), seed=3, device="cuda")
    assert open(a + "/model.safetensors", "rb").read() == open(b + "/model.safetensors", "rb").read()
