"""Bank loader on CPU: checkpoint directories written here in the two layouts the reference reads (per-expert FP4
tensors; stacked affine tensors with a config.json), indexed and loaded into a SlabBank on the host."""
import json
import struct

import numpy as np
import pytest
import torch

from oracle import configs


def _write_safetensors(path, tensors: dict):
    """tensors: name -> numpy array; a minimal writer of the format (8-byte header length, JSON header, raw bytes)."""
    code = {np.dtype(np.uint8): "U8", np.dtype(np.uint32): "U32", np.dtype(np.float16): "F16", np.dtype(np.float32): "F32"}
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        b = np.ascontiguousarray(a).tobytes()
        header[name] = {"dtype": code[a.dtype], "shape": list(a.shape), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def test_fp4_checkpoint_indexes_and_loads(tmp_path):
    from cachalot_b200 import loader
    hidden, inter, n_layers, n_exp = 64, 96, 2, 3
    rng = np.random.default_rng(0)
    experts = {(l, e): configs.fp4_expert(rng, hidden, inter) for l in range(n_layers) for e in range(n_exp)}
    del experts[(1, 2)]                                           # an expert the checkpoint lacks
    for shard, keys in enumerate(([k for k in experts if k[0] == 0], [k for k in experts if k[0] == 1]), 1):
        t = {"unrelated.weight": np.zeros(8, np.float32)}
        for (l, e) in keys:
            for name, a in experts[(l, e)].items():
                t[f"layers.{l}.ffn.experts.{e}.{name}"] = a
        _write_safetensors(tmp_path / f"model-{shard:05d}-of-00002.safetensors", t)
    (tmp_path / "model-00003-of-00003.safetensors").write_bytes(b"\\x07")     # a shard still being written is skipped
    fmt, index = loader.detect_expert_bank(tmp_path)
    assert fmt.kind == "fp4" and sorted(index) == sorted(experts)
    assert all(len(v.tensors) == 6 for v in index.values())
    bank = loader.load_bank(tmp_path, device="cpu")
    assert (bank.hidden, bank.inter, bank.layers, bank.n_experts) == (hidden, inter, n_layers, n_exp)
    assert bank.slot_table_host[1, 2] == -1 and int((bank.slot_table_host >= 0).sum()) == 5
    for (l, e), m in experts.items():
        slot = int(bank.slot_table_host[l, e])
        for name, a in m.items():
            assert np.array_equal(bank.view(slot, name).numpy(), a.reshape(-1).view(np.uint8)), (l, e, name)
    with pytest.raises(KeyError):
        bank.expert(1, 2)
    only1 = loader.load_bank(tmp_path, device="cpu", layers=[1])
    assert only1.layers == 1 and np.array_equal(only1.view(0, "w2.scale").numpy(), experts[(1, 0)]["w2.scale"].reshape(-1))
    with pytest.raises(KeyError):
        loader.load_bank(tmp_path / "nowhere", device="cpu")


def test_stacked_affine_checkpoint_indexes_and_loads(tmp_path):
    from cachalot_b200 import loader
    hidden, inter, n_exp = 128, 256, 4
    rng = np.random.default_rng(1)
    experts = [configs.affine_expert(rng, hidden, inter) for _ in range(n_exp)]
    stacked, modules = {}, {}
    for proj in ("w1", "w2", "w3"):
        modules[f"language_model.layers.5.ffn.experts.{proj}"] = {"mode": "affine", "bits": 2, "group_size": 128}
        for field in ("weight", "scales", "biases"):
            stacked[f"language_model.layers.5.ffn.experts.{proj}.{field}"] = np.stack([e[f"{proj}.{field}"] for e in experts])
    _write_safetensors(tmp_path / "model-00001-of-00001.safetensors", stacked)
    (tmp_path / "config.json").write_text(json.dumps({"omlx_deepseek_v41": {"quantized_modules": modules}}))
    fmt, index = loader.detect_expert_bank(tmp_path)
    assert (fmt.kind, fmt.bits, fmt.group_size) == ("affine", 2, 128) and sorted(index) == [(5, e) for e in range(n_exp)]
    assert fmt.tensor_names[:3] == ("w1.weight", "w1.scales", "w1.biases")
    bank = loader.load_bank(tmp_path, device="cpu")
    assert (bank.hidden, bank.inter) == (hidden, inter)
    for e, m in enumerate(experts):
        for name, a in m.items():
            assert np.array_equal(bank.view(e, name).numpy(), np.ascontiguousarray(a).reshape(-1).view(np.uint8)), (e, name)
    modules["language_model.layers.5.ffn.experts.w2"]["bits"] = 3
    (tmp_path / "config.json").write_text(json.dumps({"omlx_deepseek_v41": {"quantized_modules": modules}}))
    with pytest.raises(ValueError, match="mixed"):
        loader.detect_expert_bank(tmp_path)


def test_short_read_and_size_mismatch_are_errors(tmp_path):
    from cachalot_b200 import loader
    rng = np.random.default_rng(2)
    m = configs.fp4_expert(rng, 64, 96)
    _write_safetensors(tmp_path / "model-00001-of-00001.safetensors", {f"layers.0.ffn.experts.0.{n}": a for n, a in m.items()})
    _, index = loader.detect_expert_bank(tmp_path)
    entry = index[(0, 0)]
    views = {t.short: bytearray(t.size) for t in entry.tensors}
    assert loader.read_expert_into(entry, views, {}) == sum(t.size for t in entry.tensors)
    views["w2.weight"] = bytearray(5)
    with pytest.raises(ValueError, match="slot buffer"):
        loader.read_expert_into(entry, views, {})
    shard = tmp_path / "model-00001-of-00001.safetensors"
    data = shard.read_bytes()
    shard.write_bytes(data[:-100])                                # the file ends inside the last tensor
    views = {t.short: bytearray(t.size) for t in entry.tensors}
    with pytest.raises(OSError, match="Short read"):
        loader.read_expert_into(entry, views, {})
