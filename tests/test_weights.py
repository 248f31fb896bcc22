import json
import os
import struct

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.weights import SafetensorsError, SafetensorsFile, write_safetensors
from tests.helpers import TINY_A, make_folder


def model(dtype="float32"):
    return bb.Model(bb.Gemma2Config(**TINY_A), dtype=dtype, device="cpu")


def test_expected_tensor_names_and_shapes():
    exp = model().expected_tensors()
    assert len(exp) == 11 * 2 + 2 + 1
    assert exp["model.embed_tokens.weight"].shape == (256, 64)
    assert exp["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert exp["model.layers.0.mlp.down_proj.weight"].shape == (64, 128)
    assert exp["model.norm.weight"].role == "vector" and exp["lm_head.weight"].optional


def test_safetensors_round_trip_matches_the_reference_reader(tmp_path):
    from safetensors.torch import load_file
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors)
    theirs = load_file(path)
    ours = SafetensorsFile(path)
    for n, t in tensors.items():
        assert torch.equal(theirs[n], t) and torch.equal(ours.tensor(n), t) and ours.shape(n) == tuple(t.shape)


def test_random_folder_is_reproducible_and_seeded(tmp_path):
    cfg = bb.Gemma2Config(**TINY_A)
    for sub, seed in (("s0", 0), ("s0again", 0), ("s1", 1)):
        bb.write_random_model(cfg, str(tmp_path / sub), seed=seed)
    f0, f0b, f1 = (SafetensorsFile(str(tmp_path / s / "model.safetensors")) for s in ("s0", "s0again", "s1"))
    n = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(f0.tensor(n), f0b.tensor(n)) and not torch.equal(f0.tensor(n), f1.tensor(n))
    assert f0.dtype(n) == torch.bfloat16 and "lm_head.weight" not in f0
    assert abs(float(f0.tensor(n).float().std()) - 0.02) < 0.002
    assert abs(float(f0.tensor("model.norm.weight").float().std()) - 0.1) < 0.04
    assert json.load(open(tmp_path / "s0" / "config.json"))["architectures"] == ["Gemma2ForCausalLM"]


def test_random_values_are_a_function_of_seed_name_and_index():
    """The generator restated with Python's own integers: splitmix64 at 3 i + j + 1 steps from the key,
    twelve 16-bit fields summed, centred and scaled (brolm_b200/weights/random_init.py)."""
    import hashlib

    import numpy as np

    from brolm_b200.weights.random_init import random_tensor
    M = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    name, seed, std = "model.layers.3.mlp.up_proj.weight", 5, 0.02
    key = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")
    got = random_tensor(seed, name, (7, 9), std, torch.float32, "cpu").reshape(-1)
    for i in (0, 1, 8, 62):
        total = 0
        for j in range(3):
            z = mix((key + (3 * i + j + 1) * 0x9E3779B97F4A7C15) & M)
            total += sum((z >> s) & 0xFFFF for s in (0, 16, 32, 48))
        want = np.float32(np.float32(total - 393210) / np.float32(65536.0)) * np.float32(std)
        assert float(got[i]) == float(want)
    # a tensor does not depend on how it is cut into chunks, and looks normal
    from brolm_b200.weights import random_init
    big = random_tensor(1, "t", (1000, 300), 1.0, torch.float32, "cpu")
    old = random_init.CHUNK
    random_init.CHUNK = 4099
    try:
        assert torch.equal(random_tensor(1, "t", (1000, 300), 1.0, torch.float32, "cpu"), big)
    finally:
        random_init.CHUNK = old
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01 and float(big.abs().max()) < 6.0
    assert 0.66 < float((big.abs() < 1.0).float().mean()) < 0.70


def test_kept_element_types(tmp_path):
    folder = make_folder(tmp_path, "A", torch.bfloat16)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n) for n in f.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()          # stored in 32 bits
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].half()
    m = model("bfloat16").load_weights(tensors)
    assert m.final_norm.weight.dtype == torch.float32                            # stays 32-bit
    assert m.blocks[0].pre_mixer_norm.weight.dtype == torch.bfloat16
    assert m.embedding.dtype == torch.bfloat16 and m.head is m.embedding           # tied: the same storage
    m32 = model("float32").load_weights(tensors)
    assert m32.embedding.dtype == torch.float32 and m32.blocks[0].feedforward.w_down.dtype == torch.float32


def test_one_error_lists_everything_that_is_wrong(tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["model.layers.0.self_attn.q_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.5.extra.weight"] = torch.zeros(2)
    tensors["model.layers.1.mlp.gate_proj.weight"] = torch.zeros(64, 128)        # transposed
    with pytest.raises(bb.WeightsError) as e:
        model().load_weights(tensors)
    msg = str(e.value)
    assert "model.layers.0.self_attn.q_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.5.extra.weight" in msg and "is [64, 128], expected [128, 64]" in msg
    assert sorted(e.value.missing) == ["model.layers.0.self_attn.q_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.5.extra.weight"] and len(e.value.wrong_shape) == 1


def test_untied_model_needs_its_output_matrix(tmp_path):
    cfg = bb.Gemma2Config(**{**TINY_A, "tie_word_embeddings": False})
    m = bb.Model(cfg, dtype="float32", device="cpu")
    assert not m.expected_tensors()["lm_head.weight"].optional
    folder = make_folder(tmp_path, "A", torch.float32)               # written tied: no lm_head
    with pytest.raises(bb.WeightsError, match="lm_head.weight"):
        m.load_weights(folder)


def test_names_without_the_model_prefix_are_accepted(tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    bare = {(n[len("model."):] if n.startswith("model.") else n): f.tensor(n) for n in f.names()}
    m = model().load_weights(bare)
    assert torch.equal(m.embedding, f.tensor("model.embed_tokens.weight"))


def test_broken_files(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(p)
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", len(header)) + header + b"\0" * 8)       # payload cut short
    with pytest.raises(SafetensorsError, match="outside"):
        SafetensorsFile(p)
    (tmp_path / "empty").mkdir()
    (tmp_path / "empty" / "config.json").write_text(json.dumps({"architectures": ["Gemma2ForCausalLM"], **TINY_A}))
    with pytest.raises(SafetensorsError, match="no safetensors"):
        bb.load_model(str(tmp_path / "empty"), dtype="float32", device="cpu")
