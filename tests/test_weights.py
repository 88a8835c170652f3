"""safetensors reading and writing, the model's tensor list, and the one error for every mismatch."""
import json
import struct

import pytest
import torch

import tiny
from cpi_b200.config import spec_from_model_dir
from cpi_b200.engine.model import tensor_requirements
from cpi_b200.weights import (DictSource, SafetensorsDir, SafetensorsError, SafetensorsSource, WeightsError,
                              check_source, kept_dtype, write_safetensors, RandomSource)


def test_round_trip_and_dtypes(tmp_path):
    ts = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int64), "c": torch.randn(2, 2),
          "d": torch.randn(4).half(), "e": torch.empty(0, 3)}
    write_safetensors(str(tmp_path / "model.safetensors"), ts)
    s = SafetensorsDir(str(tmp_path))
    for k, v in ts.items():
        assert torch.equal(s.tensor(k), v) and s.entry(k).shape == tuple(v.shape)
    src = SafetensorsSource(str(tmp_path))
    assert src.get("a", "cpu").dtype == torch.bfloat16          # kept in bfloat16
    assert src.get("c", "cpu").dtype == torch.float32           # stored in 32-bit: stays so
    assert src.get("b", "cpu").dtype == torch.int32             # integer tables as int32
    assert src.get("d", "cpu").dtype == torch.float32 and torch.equal(src.get("d", "cpu"), ts["d"].float())
    assert kept_dtype(torch.bfloat16) == torch.bfloat16
    with pytest.raises(SafetensorsError, match="tensor not found: zz"):
        s.entry("zz")


def test_shards_sorted_first_name_wins(tmp_path):
    write_safetensors(str(tmp_path / "model-00002.safetensors"), {"x": torch.ones(2), "y": torch.ones(1)})
    write_safetensors(str(tmp_path / "model-00001.safetensors"), {"x": torch.zeros(2)})
    s = SafetensorsDir(str(tmp_path))
    assert torch.equal(s.tensor("x"), torch.zeros(2)) and "y" in s


def test_container_errors(tmp_path):
    with pytest.raises(SafetensorsError, match="no \\*.safetensors"):
        SafetensorsDir(str(tmp_path))
    p = tmp_path / "model.safetensors"
    write_safetensors(str(p), {"a": torch.randn(64, 64)})
    raw = p.read_bytes()
    p.write_bytes(raw[:len(raw) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsDir(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsDir(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsDir(str(tmp_path))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 12"):
        SafetensorsDir(str(tmp_path))


def test_random_model_matches_its_own_requirements():
    for name in "AB":
        d = tiny.make_model_dir(name)
        _, spec = spec_from_model_dir(d)
        src = SafetensorsSource(d)
        check_source(tensor_requirements(spec), src, spec.ignored_tensor_prefixes)
        names = set(src.names())
        p = "language_model." if name == "B" else ""
        assert (p + "lm_head.weight" in names) == (name == "A")         # B ties its head
        assert p + "model.layers.1.feed_forward.experts.gate_up_proj" in names
        assert (p + "model.layers.0.feed_forward.gate_proj.weight" in names) == (name == "B")
        norm = src.get(p + "model.layers.0.input_layernorm.weight", "cpu")
        assert norm.dtype == torch.bfloat16 and bool((norm == 1).all())
        w = src.get(p + "model.layers.1.self_attn.q_proj.weight", "cpu").float()
        std = {"A": 0.02, "B": 0.05}[name]
        assert abs(float(w.std()) - std) < 0.1 * std


def test_random_source_is_order_independent_and_seeded():
    _, spec = spec_from_model_dir(tiny.make_model_dir("A"))
    reqs = tensor_requirements(spec)
    a, b, c = RandomSource(reqs, 5, 0.02), RandomSource(reqs, 5, 0.02), RandomSource(reqs, 6, 0.02)
    name = "model.layers.1.self_attn.o_proj.weight"
    first = a.get(name, "cpu")
    for n in reversed(a.names()):
        b.get(n, "cpu")
    assert torch.equal(first, b.get(name, "cpu"))
    assert not torch.equal(first, c.get(name, "cpu"))


def test_random_draws_are_counter_based():
    """Element i of a tensor depends on (seed, name, i) alone: any cut of the stream gives the same values, and
    they are normal with the asked deviation."""
    from cpi_b200.weights.random_init import counter_normal
    x = counter_normal(777, 0, 1 << 18, 0.05, "cpu")
    assert torch.equal(counter_normal(777, 12345, 100, 0.05, "cpu"), x[12345:12445])
    assert abs(float(x.mean())) < 5e-4 and abs(float(x.std()) - 0.05) < 5e-4
    assert abs(float(((x / 0.05) ** 4).mean()) - 3.0) < 0.1          # the fourth moment of a normal
    assert abs(float((x[1:] * x[:-1]).mean())) < 2e-5                # neighbours do not correlate
    # the integer mixing against plain Python arithmetic modulo 2^64
    from cpi_b200.weights.random_init import _normal_table
    m = (1 << 64) - 1
    for i in (0, 1, 4097, (1 << 18) - 1):
        z = (i * 0x9E3779B97F4A7C15 + 777) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        z ^= z >> 31
        assert float(x[i]) == float(_normal_table()[z >> 48] * 0.05)


def test_missing_names_come_with_the_nearest_found_name(tmp_path):
    d = tiny.make_model_dir("A")
    _, spec = spec_from_model_dir(d)
    reqs = tensor_requirements(spec)
    src = SafetensorsSource(d)
    tensors = {("language_model." + n if "layers.1." in n else n): src.get(n, "cpu") for n in src.names()}
    with pytest.raises(WeightsError) as e:
        check_source(reqs, DictSource(tensors), ())
    assert ("model.layers.1.self_attn.o_proj.weight  expected shape [64, 64]  "
            "(did you mean language_model.model.layers.1.self_attn.o_proj.weight?)") in str(e.value)
    with pytest.raises(Exception, match=r"tensor not found: model\.norm\.weigth \(did you mean model\.norm\.weight\?\)"):
        src.dir.entry("model.norm.weigth")


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    d = tiny.make_model_dir("A")
    _, spec = spec_from_model_dir(d)
    reqs = tensor_requirements(spec)
    src = SafetensorsSource(d)
    tensors = {n: src.get(n, "cpu") for n in src.names()}
    del tensors["model.layers.2.self_attn.k_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.feed_forward.router.weight"] = torch.zeros(5, 64).bfloat16()
    tensors["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"][:500]
    with pytest.raises(WeightsError) as e:
        check_source(reqs, DictSource(tensors), spec.ignored_tensor_prefixes)
    err, msg = e.value, str(e.value)
    assert sorted(err.missing) == ["model.layers.2.self_attn.k_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.embed_tokens.weight",
                                                        "model.layers.1.feed_forward.router.weight"]
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "expected [4, 64], found [5, 64]",
                 "model.norm.weight  expected shape [64]"):
        assert word in msg, word


def test_vision_tensors_are_ignored_and_tied_head_tolerated():
    d = tiny.make_model_dir("B")
    _, spec = spec_from_model_dir(d)
    src = SafetensorsSource(d)
    tensors = {n: src.get(n, "cpu") for n in src.names()}
    tensors["vision_model.patch_embedding.weight"] = torch.zeros(3)
    tensors["multi_modal_projector.linear_1.weight"] = torch.zeros(3)
    check_source(tensor_requirements(spec), DictSource(tensors), spec.ignored_tensor_prefixes)
    tensors["audio_tower.x"] = torch.zeros(1)
    with pytest.raises(WeightsError, match="audio_tower.x"):
        check_source(tensor_requirements(spec), DictSource(tensors), spec.ignored_tensor_prefixes)
