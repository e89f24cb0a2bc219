"""Safetensors reading and writing, weight errors, random-weights mode."""
import json
import os
import struct

import pytest
import torch

from allpaca_b200.models import DecoderModel, resolve
from allpaca_b200.parts import BuildEnv, Workspace
from allpaca_b200.weights import (Checkpoint, SafetensorsError, SafetensorsFile, WeightError,
                                  check_names, storage_dtype, write_safetensors)
from allpaca_b200.weights.random_model import write_random_model
from helpers import TINY_A, TINY_B


def cpu_model(config):
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    env = BuildEnv(torch.float32, torch.device("cpu"), Workspace(torch.device("cpu")))
    return DecoderModel(arch.spec_builder(cfg), env)


def test_round_trip_matches_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    theirs = load_file(p)
    ours = SafetensorsFile(p)
    assert ours.metadata == {"k": "v"}
    for n in t:
        assert torch.equal(theirs[n], t[n]) and torch.equal(ours.tensor(n), t[n])
        assert ours.info(n) == (t[n].dtype, tuple(t[n].shape))
    q = str(tmp_path / "y.safetensors")
    save_file(t, q)
    assert all(torch.equal(SafetensorsFile(q).tensor(n), t[n]) for n in t)


def test_broken_files_are_named(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="overruns"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(str(p))
    h = json.dumps({"t": {"dtype": "F8", "shape": [1], "data_offsets": [0, 1]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"x")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))
    h = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"xxxx")
    with pytest.raises(SafetensorsError, match="needs 8 bytes"):
        SafetensorsFile(str(p))
    h = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"xxxx")
    with pytest.raises(SafetensorsError, match="outside"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="no model folder"):
        Checkpoint(str(tmp_path / "nowhere"))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        Checkpoint(str(empty))


def test_sharded_checkpoint_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    with pytest.raises(SafetensorsError, match="several"):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    c = Checkpoint(str(tmp_path))
    assert sorted(c.names()) == ["a", "b"] and c.tensor("b").shape == (3,)
    write_safetensors(str(tmp_path / "s2.safetensors"), {"a": torch.zeros(3)})
    with pytest.raises(SafetensorsError, match="appears in both"):
        Checkpoint(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    model = cpu_model(TINY_A)
    targets = model.weight_targets()
    have = {n: ws.shape for n, (ws, _, _) in targets.items()}
    del have["model.layers.1.mlp.up_proj.weight"]
    del have["model.norm.weight"]
    have["model.layers.0.self_attn.q_proj.bias"] = (64,)
    have["model.layers.0.self_attn.k_proj.weight"] = (64, 64)
    with pytest.raises(WeightError) as e:
        check_names(targets, have)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.norm.weight" in msg and "up_proj" in msg
    assert "unexpected tensors (1)" in msg and "q_proj.bias" in msg
    assert "wrong shapes (1)" in msg and "has [64, 64], expected [32, 64]" in msg


def test_lm_head_may_be_absent_only_as_tying():
    model = cpu_model(TINY_B)
    targets = model.weight_targets()
    have = {n: ws.shape for n, (ws, _, _) in targets.items() if n != "lm_head.weight"}
    check_names(targets, have)        # tied by absence: fine


def test_storage_types():
    assert storage_dtype(torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float16, torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float32, torch.bfloat16) == torch.float32   # stays 32-bit
    assert storage_dtype(torch.int64, torch.bfloat16) == torch.int32


def test_random_weights_are_seeded_and_shaped(tmp_path):
    a, b, c = (str(tmp_path / x) for x in "abc")
    write_random_model(a, TINY_B, 1, "float32", norm_std=0.02)
    write_random_model(b, TINY_B, 1, "float32", norm_std=0.02)
    write_random_model(c, TINY_B, 2, "bfloat16")
    ca, cb, cc = Checkpoint(a), Checkpoint(b), Checkpoint(c)
    assert "lm_head.weight" not in ca                     # tied
    assert all(torch.equal(ca.tensor(n), cb.tensor(n)) for n in ca.names())
    assert not torch.equal(ca.tensor("model.embed_tokens.weight").to(torch.bfloat16),
                           cc.tensor("model.embed_tokens.weight"))
    w = ca.tensor("model.layers.2.mlp.down_proj.weight")
    assert w.shape == (96, 256) and abs(float(w.std()) - 0.02) < 0.002
    n = ca.tensor("model.layers.0.input_layernorm.weight")
    assert abs(float(n.mean()) - 1.0) < 0.02 and float(n.std()) > 0.005
    assert torch.equal(cc.tensor("model.norm.weight"), torch.ones(96, dtype=torch.bfloat16))
    assert json.load(open(os.path.join(c, "config.json")))["torch_dtype"] == "bfloat16"
    check_names(cpu_model(TINY_B).weight_targets(), {n: ca.info(n)[1] for n in ca.names()})


def _file_with_header(path, header_bytes, data=b""):
    path.write_bytes(struct.pack("<Q", len(header_bytes)) + header_bytes + data)
    return str(path)


def test_native_reader_header_corner_cases(tmp_path):
    """The C++ reader of the header: escapes and non-ASCII in names, metadata, whitespace,
    tensors without elements, names written twice, bytes that are not UTF-8, entries that
    are not what they should be."""
    p = tmp_path / "h.safetensors"
    data = struct.pack("<4f", 1.0, 2.0, 3.0, 4.0)
    h = ('{ "__metadata__": {"format": "pt", "n\\u00e4me": "caf\\u00e9 \\ud83d\\ude00"},\n'
         ' "layer\\u002e0.w\\/x": {"dtype":"F32","shape":[2,2],"data_offsets":[0,16]},\n'
         ' "größe": {"dtype":"BF16","shape":[0,7],"data_offsets":[16,16]},\n'
         ' "scalar": {"dtype":"F32","shape":[],"data_offsets":[12,16]} }   ').encode("utf-8")
    f = SafetensorsFile(_file_with_header(p, h, data))
    assert f.metadata == {"format": "pt", "näme": "café \U0001F600"}
    assert f.names() == ["layer.0.w/x", "größe", "scalar"]
    assert torch.equal(f.tensor("layer.0.w/x"), torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    assert f.info("größe") == (torch.bfloat16, (0, 7)) and f.tensor("größe").shape == (0, 7)
    assert f.tensor("scalar").shape == () and float(f.tensor("scalar")) == 4.0

    twice = b'{"t":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},"t":{"dtype":"U8","shape":[1],"data_offsets":[0,1]}}'
    with pytest.raises(SafetensorsError, match="appears twice"):
        SafetensorsFile(_file_with_header(p, twice, b"x"))
    with pytest.raises(SafetensorsError, match="not UTF-8"):
        SafetensorsFile(_file_with_header(p, b'{"t\xff": 1}'))
    with pytest.raises(SafetensorsError, match="not a JSON object"):
        SafetensorsFile(_file_with_header(p, b'[1, 2]'))
    with pytest.raises(SafetensorsError, match="not JSON.*text after the value"):
        SafetensorsFile(_file_with_header(p, b'{} {}'))
    for bad in (b'{"t": 3}', b'{"t":{"dtype":"F32","shape":[1.5],"data_offsets":[0,4]}}',
                b'{"t":{"dtype":"F32","shape":[-1],"data_offsets":[0,4]}}',
                b'{"t":{"dtype":"F32","shape":[1],"data_offsets":[0]}}',
                b'{"t":{"dtype":7,"shape":[1],"data_offsets":[0,4]}}'):
        with pytest.raises(SafetensorsError, match="malformed entry for tensor 't'"):
            SafetensorsFile(_file_with_header(p, bad, b"xxxx"))
    huge = b'{"t":{"dtype":"F64","shape":[4294967296,4294967296],"data_offsets":[0,8]}}'
    with pytest.raises(SafetensorsError, match="needs more than"):
        SafetensorsFile(_file_with_header(p, huge, b"x" * 8))
    with pytest.raises(SafetensorsError, match="header length 0"):
        p.write_bytes(struct.pack("<Q", 0) + b"{}")
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "missing.safetensors"))


def test_a_tensor_keeps_its_mapping_alive(tmp_path):
    import gc
    p = str(tmp_path / "x.safetensors")
    want = torch.arange(1000, dtype=torch.float32)
    write_safetensors(p, {"w": want})
    t = SafetensorsFile(p).tensor("w")          # the file object itself is dropped at once
    gc.collect()
    os.remove(p)
    assert torch.equal(t, want) and torch.equal(t[10:20].clone(), want[10:20])


def test_native_header_reader_agrees_with_json_on_random_headers(tmp_path):
    """Names of any characters, written escaped or raw, with any spacing: the C++ reader and
    Python's json module read the same entries, in the same order."""
    from hypothesis import given, settings, strategies as st
    p = tmp_path / "r.safetensors"
    chars = st.characters(blacklist_categories=("Cs",), blacklist_characters="\0")
    names = st.text(chars, min_size=1, max_size=12).filter(lambda n: n != "__metadata__")
    shapes = st.lists(st.integers(0, 5), max_size=3)

    @settings(max_examples=60, deadline=None)
    @given(st.dictionaries(names, shapes, max_size=6), st.booleans(), st.sampled_from([None, 1, 3]),
           st.dictionaries(st.text(chars, max_size=6), st.text(chars, max_size=6), max_size=3))
    def check(tensors, ascii_only, indent, meta):
        header, offset = {}, 0
        if meta:
            header["__metadata__"] = meta
        for name, shape in tensors.items():
            n = 2
            for s in shape:
                n *= s
            header[name] = {"dtype": "BF16", "shape": shape, "data_offsets": [offset, offset + n]}
            offset += n
        raw = json.dumps(header, ensure_ascii=ascii_only, indent=indent).encode("utf-8")
        f = SafetensorsFile(_file_with_header(p, raw, b"\0" * offset))
        assert f.names() == list(tensors)
        assert f.metadata == (meta or {})
        for name, shape in tensors.items():
            assert f.info(name) == (torch.bfloat16, tuple(shape))
            assert f.tensor(name).shape == tuple(shape)
    check()
    with pytest.raises(SafetensorsError, match="NUL"):
        SafetensorsFile(_file_with_header(p, b'{"a\\u0000b":{"dtype":"U8","shape":[0],"data_offsets":[0,0]}}'))


def test_matrices_stored_in_32_bit_under_a_bfloat16_engine(tmp_path, capsys):
    """A 32-bit checkpoint loaded for a bfloat16 engine: kept (and said aloud, because such
    matrices run on the slow CUDA-core product), rounded, or refused; norm weights stay 32-bit
    in every case; a bfloat16 checkpoint says nothing."""
    from allpaca_b200.weights import load_checkpoint
    d32, d16 = str(tmp_path / "f32"), str(tmp_path / "bf16")
    write_random_model(d32, TINY_A, 0, "float32", norm_std=0.02)
    write_random_model(d16, TINY_A, 0, "bfloat16", norm_std=0.02)
    cpu = torch.device("cpu")

    def load(path, policy):
        model = cpu_model(TINY_A)
        load_checkpoint(model, path, torch.bfloat16, cpu, policy)
        block = model.blocks[0]
        return block.mixer.qkv.weight.dtype, block.mixer_norm.weight.dtype, model.embedding.dtype

    assert load(d32, "keep") == (torch.float32, torch.float32, torch.float32)
    said = capsys.readouterr().err
    assert "stored in 32-bit" in said and "CUDA cores" in said
    assert load(d32, "round") == (torch.bfloat16, torch.float32, torch.bfloat16)
    assert capsys.readouterr().err == ""
    with pytest.raises(WeightError, match="stored in 32-bit"):
        load(d32, "refuse")
    assert load(d16, "keep") == (torch.bfloat16, torch.bfloat16, torch.bfloat16)
    assert capsys.readouterr().err == ""
    with pytest.raises(WeightError, match="float32_weights"):
        load(d16, "sometimes")
