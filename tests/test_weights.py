import os
import shutil

import pytest
import torch

import tiny_configs
from distengine_b200.models.decoder import expected_tensors
from distengine_b200.registry import read_config
from distengine_b200.weights import WeightMismatchError, load_checked, save_tensors
from distengine_b200.weights.safetensors_io import SafetensorsFile


def _expected(folder):
    _, config = read_config(folder)
    return expected_tensors(config)


def test_random_model_folder_is_reproducible_and_readable(model_root, tmp_path):
    a = tiny_configs.make_folder("tiny_a", model_root)
    b = tiny_configs.make_folder("tiny_a", str(tmp_path))
    expected, vectors, optional = _expected(a)
    ta, tb = load_checked(a, expected, optional, torch.float32), load_checked(b, expected, optional,
                                                                              torch.float32)
    assert set(ta) == set(expected)
    for name in expected:
        assert torch.equal(ta[name], tb[name]) and tuple(ta[name].shape) == expected[name]
    assert all(torch.all(ta[n] == 1) for n in vectors)                  # norm weights are ones
    w = ta["model.layers.0.mlp.down_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    # the library reads the file the same way
    from safetensors.torch import load_file
    theirs = load_file(os.path.join(a, "model.safetensors"))
    assert all(torch.equal(theirs[n], ta[n]) for n in expected)


def test_tied_model_has_no_output_matrix_and_uniform_norms(model_root):
    folder = tiny_configs.make_folder("tiny_b", model_root)
    expected, vectors, optional = _expected(folder)
    assert optional == {"lm_head.weight"}
    tensors = load_checked(folder, expected, optional, torch.float32)
    assert "lm_head.weight" not in tensors
    norm = tensors["model.norm.weight"]
    assert 0.5 <= norm.min() and norm.max() <= 1.5 and norm.std() > 0.1


def test_dtypes_stay_as_stored(tmp_path):
    tensors = {"a": torch.randn(4, 4).to(torch.bfloat16), "b": torch.randn(4),
               "c": torch.randn(2, 2).to(torch.float16), "d": torch.arange(6, dtype=torch.int64)}
    os.makedirs(tmp_path / "m")
    save_tensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    expected = {k: tuple(v.shape) for k, v in tensors.items()}
    kept = load_checked(str(tmp_path / "m"), expected, dtype=torch.bfloat16, integer={"d"})
    assert kept["a"].dtype == torch.bfloat16 and torch.equal(kept["a"], tensors["a"])
    assert kept["b"].dtype == torch.float32 and torch.equal(kept["b"], tensors["b"])   # 32-bit stays
    assert kept["c"].dtype == torch.bfloat16
    assert kept["d"].dtype == torch.int32 and kept["d"].tolist() == list(range(6))
    wide = load_checked(str(tmp_path / "m"), expected, dtype=torch.float32, integer={"d"})
    assert wide["a"].dtype == wide["c"].dtype == torch.float32 and wide["d"].dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_root, tmp_path):
    src = tiny_configs.make_folder("tiny_a", model_root)
    expected, _, optional = _expected(src)
    handle = SafetensorsFile(os.path.join(src, "model.safetensors"))
    tensors = {n: handle.tensor(n).clone() for n in handle.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)       # ignored
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64)
    dst = tmp_path / "broken"
    os.makedirs(dst)
    shutil.copy(os.path.join(src, "config.json"), dst / "config.json")
    save_tensors(str(dst / "model.safetensors"), tensors)
    with pytest.raises(WeightMismatchError) as info:
        load_checked(str(dst), expected, optional, torch.float32)
    err = info.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (64, 64))]
    text = str(err)
    for piece in ("missing tensors (2)", "model.norm.weight", "unexpected tensors (1)",
                  "q_proj.bias", "wrong shapes (1)", "expected [32, 64], file has [64, 64]"):
        assert piece in text


def test_a_tensor_of_the_wrong_class_of_dtype_is_named(model_root, tmp_path):
    """Integers or booleans under a matrix's or a norm weight's name are not cast and loaded: the
    error names them; so is a floating-point tensor where an integer table is expected."""
    src = tiny_configs.make_folder("tiny_a", model_root)
    expected, _, optional = _expected(src)
    handle = SafetensorsFile(os.path.join(src, "model.safetensors"))
    tensors = {n: handle.tensor(n).clone() for n in handle.names()}
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.ones(64, 176, dtype=torch.int8)
    tensors["model.norm.weight"] = torch.ones(64, dtype=torch.bool)
    dst = tmp_path / "ints"
    os.makedirs(dst)
    shutil.copy(os.path.join(src, "config.json"), dst / "config.json")
    save_tensors(str(dst / "model.safetensors"), tensors)
    with pytest.raises(WeightMismatchError) as info:
        load_checked(str(dst), expected, optional, torch.bfloat16)
    err = info.value
    assert [name for name, _, _ in err.wrong_dtype] == ["model.layers.0.mlp.down_proj.weight",
                                                        "model.norm.weight"]
    assert not err.missing and not err.unexpected and not err.wrong_shape
    assert "model.norm.weight: expected a floating-point dtype, file has torch.bool" in str(err)
    with pytest.raises(WeightMismatchError, match="expected an integer dtype"):
        load_checked(str(dst), expected, optional, torch.bfloat16,
                     integer={"model.layers.1.mlp.up_proj.weight"})


def test_a_folder_of_shards_is_read_through_its_index(model_root, tmp_path):
    """model.safetensors.index.json names the files; every tensor is found in its shard, a tensor
    that no shard holds is missing, and a shard's extra tensor is unexpected."""
    import json
    src = tiny_configs.make_folder("tiny_a", model_root)
    expected, _, optional = _expected(src)
    handle = SafetensorsFile(os.path.join(src, "model.safetensors"))
    names = handle.names()
    parts = [names[0::3], names[1::3], names[2::3]]
    dst = tmp_path / "shards"
    os.makedirs(dst)
    weight_map = {}
    for i, part in enumerate(parts):
        file = f"model-{i + 1:05d}-of-00003.safetensors"
        save_tensors(str(dst / file), {n: handle.tensor(n).clone() for n in part})
        weight_map.update({n: file for n in part})
    with open(dst / "model.safetensors.index.json", "w") as out:
        json.dump({"metadata": {}, "weight_map": weight_map}, out)
    whole = load_checked(src, expected, optional, torch.float32)
    sharded = load_checked(str(dst), expected, optional, torch.float32)
    assert set(sharded) == set(whole) and all(torch.equal(sharded[n], whole[n]) for n in whole)
    # one shard loses a tensor and gains a stranger
    file = f"model-{2:05d}-of-00003.safetensors"
    kept = {n: handle.tensor(n).clone() for n in parts[1][1:]}
    kept["model.stranger"] = torch.zeros(3)
    save_tensors(str(dst / file), kept)
    with pytest.raises(WeightMismatchError) as info:
        load_checked(str(dst), expected, optional, torch.float32)
    assert info.value.missing == [parts[1][0]] and info.value.unexpected == ["model.stranger"]


def test_untied_model_without_output_matrix_is_an_error(model_root, tmp_path):
    src = tiny_configs.make_folder("tiny_a", model_root)
    expected, _, optional = _expected(src)
    handle = SafetensorsFile(os.path.join(src, "model.safetensors"))
    tensors = {n: handle.tensor(n).clone() for n in handle.names() if n != "lm_head.weight"}
    os.makedirs(tmp_path / "m")
    save_tensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    with pytest.raises(WeightMismatchError, match="lm_head.weight"):
        load_checked(str(tmp_path / "m"), expected, optional, torch.float32)


def test_not_a_safetensors_file(tmp_path):
    os.makedirs(tmp_path / "m")
    (tmp_path / "m" / "model.safetensors").write_bytes(b"\x00" * 4)
    with pytest.raises(ValueError, match="not a safetensors file"):
        load_checked(str(tmp_path / "m"), {})
    with pytest.raises(FileNotFoundError):
        load_checked(str(tmp_path / "nothing"), {})
