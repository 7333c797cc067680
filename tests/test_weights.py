"""The safetensors reader and writer, binding errors, and the random-weights mode."""
import json
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_folder
from stratakv_b200.config import LlamaConfig
from stratakv_b200.config.registry import resolve_architecture
from stratakv_b200.engine.model import expected_tensors
from stratakv_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_checkpoint,
                                   read_checkpoint, write_safetensors)


def raw_file(path, header, payload=b""):
    text = header if isinstance(header, bytes) else json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + payload)
    return path


def test_round_trip_keeps_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16),
               "c": torch.randn(7).to(torch.float16), "i": torch.arange(6, dtype=torch.int64).view(2, 3),
               "empty": torch.zeros(0, 4), "scalar": torch.tensor(2.5)}
    write_safetensors(tmp_path / "x.safetensors", tensors, {"format": "pt"})
    handle = SafetensorsFile(tmp_path / "x.safetensors")
    assert handle.metadata == {"format": "pt"} and set(handle.names()) == set(tensors)
    for name, tensor in tensors.items():
        got = handle.tensor(name)
        assert got.dtype == tensor.dtype and tuple(got.shape) == tuple(tensor.shape) and torch.equal(got, tensor)
    from safetensors import safe_open          # the file is also readable by the usual library
    with safe_open(str(tmp_path / "x.safetensors"), framework="pt") as other:
        assert torch.equal(other.get_tensor("b"), tensors["b"])


def test_views_are_private(tmp_path):
    """Writing into a loaded tensor never reaches the file (tests/phase5_smoke.cpp:94-106)."""
    write_safetensors(tmp_path / "x.safetensors", {"a": torch.ones(4)})
    first = SafetensorsFile(tmp_path / "x.safetensors").tensor("a")
    first[0] = 9.0
    assert SafetensorsFile(tmp_path / "x.safetensors").tensor("a")[0] == 1.0


def test_bfloat16_alias(tmp_path):
    path = raw_file(tmp_path / "x.safetensors", {"t": {"dtype": "bfloat16", "shape": [2], "data_offsets": [0, 4]}},
                    torch.tensor([1.0, -2.0]).to(torch.bfloat16).view(torch.uint8).numpy().tobytes())
    assert SafetensorsFile(path).tensor("t").tolist() == [1.0, -2.0]


@pytest.mark.parametrize("header,payload,message", [
    (b"{not json", b"", "not valid JSON"),
    (b"\xff\xfe{}", b"", "UTF-8"),
    ([1, 2], b"", "JSON object"),
    ({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4, "does not hold"),
    ({"t": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4, "unsupported dtype"),
    ({"t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4], "extra": 1}}, b"\0" * 4, "unknown field"),
    ({"t": {"dtype": "F32", "shape": [1]}}, b"\0" * 4, "missing 'data_offsets'"),
    ({"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 4, "non-negative"),
    ({"t": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}, b"\0" * 4, "does not hold"),
    ({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "payload has 4"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
      "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 6, "overlaps"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8, "belong to no tensor"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 8, "belong to no tensor"),
    ({"__metadata__": {"k": 1}}, b"", "__metadata__"),
    (b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}, "a": {"dtype": "F32", "shape": [1], '
     b'"data_offsets": [0, 4]}}', b"\0" * 4, "duplicate key"),
])
def test_malformed_files_are_rejected(tmp_path, header, payload, message):
    """The malformed-header list of the reference's loader tests (tests/phase5_smoke.cpp:140-161)."""
    with pytest.raises(SafetensorsError, match=message):
        SafetensorsFile(raw_file(tmp_path / "bad.safetensors", header, payload))


def test_short_and_oversized_headers(tmp_path):
    (tmp_path / "short.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsFile(tmp_path / "short.safetensors")
    (tmp_path / "long.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(tmp_path / "long.safetensors")
    (tmp_path / "past.safetensors").write_bytes(struct.pack("<Q", 100) + b"{}")
    with pytest.raises(SafetensorsError, match="past the end"):
        SafetensorsFile(tmp_path / "past.safetensors")


def expected_shapes(raw):
    config = LlamaConfig.from_dict(raw)
    spec = resolve_architecture(config.architecture).build_spec(config)
    return spec, {name: request.shape for name, request in expected_tensors(spec).items()}


def test_random_model_folder_binds(tmp_path):
    for raw, dtype in ((TINY_A, torch.float32), (TINY_B, torch.bfloat16)):
        folder = make_folder(tmp_path / f"m{raw['hidden_size']}", raw, seed=3, dtype=dtype)
        spec, shapes = expected_shapes(raw)
        tensors = load_checkpoint(folder, shapes, spec.ignorable)
        assert set(tensors) == set(shapes)
        assert all(t.dtype == dtype for t in tensors.values())          # stored dtype is kept
        assert ("lm_head.weight" in shapes) == (not raw["tie_word_embeddings"])
        norm = tensors["model.norm.weight"].float()
        assert abs(norm.mean() - 1.0) < 0.02 and 0.005 < norm.std() < 0.04
        matrix = tensors["model.layers.0.mlp.gate_proj.weight"].float()
        assert abs(matrix.mean()) < 0.002 and 0.017 < matrix.std() < 0.023
        assert json.loads((folder / "config.json").read_text())["hidden_size"] == raw["hidden_size"]


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = read_checkpoint(make_folder(tmp_path / "a", TINY_A, seed=1))
    b = read_checkpoint(make_folder(tmp_path / "b", TINY_A, seed=1))
    c = read_checkpoint(make_folder(tmp_path / "c", TINY_A, seed=2))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])


def test_one_error_lists_everything(tmp_path):
    folder = make_folder(tmp_path / "m", TINY_A, seed=3)
    tensors = dict(read_checkpoint(folder))
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)       # ignorable buffer
    tensors["surprise.weight"] = torch.zeros(2)
    tensors["another.bias"] = torch.zeros(2)
    write_safetensors(folder / "model.safetensors", tensors)
    spec, shapes = expected_shapes(TINY_A)
    with pytest.raises(WeightError) as info:
        load_checkpoint(folder, shapes, spec.ignorable)
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["another.bias", "surprise.weight"]
    assert error.wrong_shape == {"model.layers.0.self_attn.k_proj.weight": ((32, 64), (16, 64))}
    text = str(error)
    for needle in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (1)", "surprise.weight",
                   "expected [32, 64] found [16, 64]"):
        assert needle in text


def test_tied_model_ignores_a_stored_head(tmp_path):
    folder = make_folder(tmp_path / "m", TINY_B, seed=3)
    tensors = dict(read_checkpoint(folder))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(folder / "model.safetensors", tensors)
    spec, shapes = expected_shapes(TINY_B)
    assert "lm_head.weight" not in load_checkpoint(folder, shapes, spec.ignorable)


def test_integer_tables_become_int32(tmp_path):
    from stratakv_b200.weights import check_and_select
    picked = check_and_select("x", {"table": torch.arange(4, dtype=torch.int64)}, {"table": (4,)})
    assert picked["table"].dtype == torch.int32


@pytest.mark.parametrize("dtype,bad", [(torch.float32, float("nan")), (torch.bfloat16, float("inf")),
                                       (torch.float32, float("-inf"))])
def test_a_non_finite_weight_is_refused_by_name(tmp_path, dtype, bad):
    """src/generation/generator.cpp:274-285: "Non-finite weight: <name>"; here it joins the one error."""
    folder = make_folder(tmp_path / "m", TINY_A, seed=3, dtype=dtype)
    tensors = {name: tensor.clone() for name, tensor in read_checkpoint(folder).items()}
    tensors["model.layers.1.mlp.down_proj.weight"][5, 7] = bad
    tensors["model.norm.weight"][0] = bad
    del tensors["lm_head.weight"]
    write_safetensors(folder / "model.safetensors", tensors)
    spec, shapes = expected_shapes(TINY_A)
    with pytest.raises(WeightError) as info:
        load_checkpoint(folder, shapes, spec.ignorable)
    assert info.value.non_finite == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert info.value.missing == ["lm_head.weight"]
    assert "non-finite weights (2): model.layers.1.mlp.down_proj.weight, model.norm.weight" in str(info.value)


def shard(folder, tensors, parts):
    """Rewrite a folder's checkpoint as ``parts`` shards with an index, the way large checkpoints ship."""
    names = sorted(tensors)
    weight_map = {}
    for part in range(parts):
        file_name = f"model-{part + 1:05d}-of-{parts:05d}.safetensors"
        mine = {name: tensors[name] for name in names[part::parts]}
        write_safetensors(folder / file_name, mine)
        weight_map.update({name: file_name for name in mine})
    (folder / "model.safetensors").unlink()
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    return weight_map


def test_a_sharded_folder_round_trips(tmp_path):
    folder = make_folder(tmp_path / "m", TINY_B, seed=4, dtype=torch.bfloat16)
    whole = {name: tensor.clone() for name, tensor in read_checkpoint(folder).items()}
    shard(folder, whole, 3)
    spec, shapes = expected_shapes(TINY_B)
    loaded = load_checkpoint(folder, shapes, spec.ignorable)
    assert set(loaded) == set(shapes)
    assert all(torch.equal(loaded[name], whole[name]) for name in loaded)


def test_a_tensor_in_two_shards_is_refused(tmp_path):
    folder = make_folder(tmp_path / "m", TINY_A, seed=4)
    whole = {name: tensor.clone() for name, tensor in read_checkpoint(folder).items()}
    weight_map = shard(folder, whole, 2)
    first, second = sorted(set(weight_map.values()))
    copied = next(name for name, file_name in weight_map.items() if file_name == first)
    again = {name: whole[name] for name, file_name in weight_map.items() if file_name == second}
    again[copied] = whole[copied]
    write_safetensors(folder / second, again)
    with pytest.raises(SafetensorsError, match="more than one shard"):
        read_checkpoint(folder)


def test_a_missing_shard_is_named(tmp_path):
    folder = make_folder(tmp_path / "m", TINY_A, seed=4)
    whole = {name: tensor.clone() for name, tensor in read_checkpoint(folder).items()}
    weight_map = shard(folder, whole, 2)
    gone = sorted(set(weight_map.values()))[1]
    (folder / gone).unlink()
    with pytest.raises(SafetensorsError, match=gone):
        read_checkpoint(folder)
