"""Weights: safetensors by name, stored precision, one error for everything wrong (no GPU)."""
import json
import os
import struct

import pytest
import torch

import helpers as H
from binfer_b200.config import Qwen3Config
from binfer_b200.parts.model import param_specs_for
from binfer_b200.weights import (ParamSpec, SafetensorsError, TensorSource, WeightError,
                                 check_names, place, random_tensors, read_header, save_file,
                                 write_model_dir)


def test_safetensors_round_trip_and_stored_precision(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "h": torch.randn(4).half()}
    path = str(tmp_path / "x.safetensors")
    save_file(t, path)
    info = read_header(path)
    assert info["a"].dtype == "F32" and info["b"].dtype == "BF16" and info["c"].shape == (2, 3)
    os.rename(path, str(tmp_path / "model.safetensors"))
    src = TensorSource.from_dir(str(tmp_path))
    assert torch.equal(src.get("a"), t["a"]) and src.get("a").dtype == torch.float32
    assert torch.equal(src.get("b"), t["b"]) and src.get("b").dtype == torch.bfloat16
    assert src.get("c").dtype == torch.int32 and src.get("c").tolist() == [[0, 1, 2], [3, 4, 5]]
    assert src.get("h").dtype == torch.bfloat16
    src.close()


def test_cross_check_with_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 4).to(torch.bfloat16), "v": torch.randn(9)}
    save_file(t, str(tmp_path / "ours.safetensors"))
    back = st.load_file(str(tmp_path / "ours.safetensors"))
    assert torch.equal(back["w"], t["w"]) and torch.equal(back["v"], t["v"])
    st.save_file(t, str(tmp_path / "model.safetensors"))
    src = TensorSource.from_dir(str(tmp_path))
    assert torch.equal(src.get("w"), t["w"])
    src.close()


def test_bad_files(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_header(p)
    with open(p, "wb") as f:
        js = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
        f.write(struct.pack("<Q", len(js)) + js + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="spans 8 bytes"):
        read_header(p)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="No safetensors files"):
        TensorSource.from_dir(str(empty))


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    specs = [ParamSpec("a", (2, 3)), ParamSpec("b", (4,)), ParamSpec("c", (5,))]
    with pytest.raises(WeightError) as e:
        check_names(specs, {"a": (3, 2), "c": (5,), "zzz": (1,), "opt": (1,)}, optional=["opt"],
                    where="somewhere")
    msg = str(e.value)
    assert "missing tensors (1): b" in msg
    assert "unexpected tensors (1): zzz" in msg
    assert "a is [3, 2], expected [2, 3]" in msg
    assert e.value.missing == ["b"] and e.value.unexpected == ["zzz"]
    check_names(specs, {"a": (2, 3), "b": (4,), "c": (5,), "opt": (1,)}, optional=["opt"])


def test_model_folder_has_every_tensor_by_its_name(tmp_path):
    d = H.make_model_dir(tmp_path, "B")
    raw, w = H.read_model_dir(d)
    assert raw["architectures"] == ["Qwen3ForCausalLM"]
    names = {s.name: s.shape for s in param_specs_for(Qwen3Config.from_dict(raw).to_spec())}
    assert set(w) == set(names)
    assert names["model.layers.2.self_attn.q_proj.weight"] == (192, 96)
    assert names["model.layers.0.self_attn.k_norm.weight"] == (32,)
    assert names["lm_head.weight"] == (300, 96)
    a = H.make_model_dir(tmp_path, "A")
    assert "lm_head.weight" not in H.read_model_dir(a)[1]          # tied


def test_random_weights_depend_on_seed_and_name_only():
    specs = param_specs_for(Qwen3Config.from_dict(H.TINY_A).to_spec())
    one = random_tensors(specs, seed=3, std=0.02, norm_std=0.01)
    two = random_tensors(list(reversed(specs)), seed=3, std=0.02, norm_std=0.01)
    assert all(torch.equal(one[k], two[k]) for k in one)
    other = random_tensors(specs, seed=4)
    assert not torch.equal(one["model.embed_tokens.weight"], other["model.embed_tokens.weight"])
    n = one["model.norm.weight"]
    assert abs(float(n.mean()) - 1) < 0.01 and float(n.std()) < 0.02
    assert abs(float(one["model.embed_tokens.weight"].std()) - 0.02) < 0.002


def test_place_keeps_32_bit_vectors_and_casts_matrices():
    cpu = torch.device("cpu")
    m, v = ParamSpec("m", (2, 2)), ParamSpec("v", (2,), role="vector")
    bf = torch.ones(2, 2, dtype=torch.bfloat16)
    assert place(bf, m, torch.bfloat16, cpu).dtype == torch.bfloat16
    assert place(bf, m, torch.float32, cpu).dtype == torch.float32
    assert place(torch.ones(2), v, torch.bfloat16, cpu).dtype == torch.float32
    assert place(torch.ones(2, dtype=torch.bfloat16), v, torch.bfloat16, cpu).dtype == torch.float32
    assert place(torch.ones(2, dtype=torch.int64), v, torch.bfloat16, cpu).dtype == torch.int32


def test_loading_a_wrong_checkpoint_fails_before_anything_is_taken(tmp_path):
    from binfer_b200.parts import BuildEnv, DecoderModel
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    del w["model.layers.1.mlp.up_proj.weight"]
    w["model.layers.0.self_attn.q_norm.weight"] = torch.ones(8)
    w["extra.bias"] = torch.zeros(1)
    model = DecoderModel(Qwen3Config.from_dict(raw).to_spec(),
                         BuildEnv(torch.float32, torch.device("cpu")))
    with pytest.raises(WeightError) as e:
        model.load(TensorSource.from_dict(w))
    assert "up_proj" in str(e.value) and "extra.bias" in str(e.value) and "[8]" in str(e.value)
    assert model.embed is None


def test_index_names_the_shards(tmp_path):
    """With model.safetensors.index.json the model is the shards it names: a missing shard
    is one error that names it, a file it does not name is ignored with a warning, and a
    tensor it names must be in its shard."""
    import warnings
    from binfer_b200.weights.loader import find_safetensors_files
    a = {"x": torch.randn(2, 2), "y": torch.randn(3)}
    b = {"z": torch.randn(4)}
    save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    index = {"metadata": {}, "weight_map": {"x": "model-00001-of-00002.safetensors",
                                            "y": "model-00001-of-00002.safetensors",
                                            "z": "model-00002-of-00002.safetensors"}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    src = TensorSource.from_dir(str(tmp_path))
    assert set(src.shapes) == {"x", "y", "z"} and torch.equal(src.get("z"), b["z"])
    src.close()
    # a stale file beside the shards is not part of the model
    save_file({"old": torch.zeros(1)}, str(tmp_path / "leftover.safetensors"))
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        src = TensorSource.from_dir(str(tmp_path))
        src.close()
    assert "old" not in src.shapes and any("leftover.safetensors" in str(x.message) for x in w)
    # a tensor the index promises but the shard lacks
    index["weight_map"]["gone"] = "model-00002-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightError, match="gone"):
        TensorSource.from_dir(str(tmp_path))
    # a shard that is not there
    os.remove(str(tmp_path / "model-00002-of-00002.safetensors"))
    with pytest.raises(FileNotFoundError, match="model-00002-of-00002.safetensors"):
        find_safetensors_files(str(tmp_path))


def test_unexpected_tensors_can_be_a_warning():
    import warnings
    specs = [ParamSpec("a", (2, 3))]
    with pytest.raises(WeightError, match="unexpected tensors"):
        check_names(specs, {"a": (2, 3), "buffer": (1,)})
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        check_names(specs, {"a": (2, 3), "buffer": (1,)}, allow_unexpected=True)
    assert any("buffer" in str(x.message) for x in w)
    # what is missing or misshapen stays an error, and the error still lists the extras
    with pytest.raises(WeightError) as e:
        check_names(specs, {"a": (3, 2), "buffer": (1,)}, allow_unexpected=True)
    assert "buffer" in str(e.value) and "expected [2, 3]" in str(e.value)
