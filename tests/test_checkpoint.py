"""Prepacked checkpoint directory: round trip, and loud failures on damaged or foreign content (CPU)."""

import json
import os

import numpy as np
import pytest
import torch

from liquidgemm_b200 import checkpoint as C


def _layer(N, K, seed):
    g = torch.Generator().manual_seed(seed)
    return {"rs": torch.randint(0, 256, (C.blob_bytes(N, K),), dtype=torch.uint8, generator=g),
            "s1": torch.rand(N, generator=g), "s_u8": torch.randint(1, 17, (N, K // 64), dtype=torch.uint8, generator=g),
            "offset_a": torch.randint(0, 256, (N, K // 64), dtype=torch.uint8, generator=g), "N": N, "K": K}


def test_round_trip(tmp_path):
    layers = [("model.layers.0.qkv", _layer(192, 256, 1)), ("model.layers.0.down", _layer(100, 128, 2))]
    cfg_path = C.save_prepacked(str(tmp_path), layers)
    assert os.path.basename(cfg_path) == C.CONFIG_NAME
    got = C.load_prepacked(str(tmp_path))
    assert list(got) == [n for n, _ in layers]
    for name, L in layers:
        for k in ("rs", "s1", "s_u8", "offset_a"):
            assert torch.equal(got[name][k], L[k]), (name, k)
        assert (got[name]["N"], got[name]["K"]) == (L["N"], L["K"])
    cfg = C.read_config(str(tmp_path))
    assert cfg["quant_method"] == "liquidgemm" and cfg["group_size"] == 64 and cfg["version"] == C.VERSION


def test_blob_size_is_checked_on_save(tmp_path):
    bad = _layer(128, 256, 3)
    bad["rs"] = bad["rs"][:-1]
    with pytest.raises(ValueError):
        C.save_prepacked(str(tmp_path), [("x", bad)])


def test_damaged_file_and_foreign_config_fail_loudly(tmp_path):
    C.save_prepacked(str(tmp_path), [("a", _layer(128, 128, 4))])
    f = os.path.join(str(tmp_path), "00000.lqq")
    data = bytearray(open(f, "rb").read())
    data[-1] ^= 0xFF
    open(f, "wb").write(bytes(data))
    with pytest.raises(ValueError):
        C.load_prepacked(str(tmp_path))
    cfgp = os.path.join(str(tmp_path), C.CONFIG_NAME)
    cfg = json.load(open(cfgp))
    cfg["version"] = 99
    json.dump(cfg, open(cfgp, "w"))
    with pytest.raises(ValueError):
        C.read_config(str(tmp_path))


def test_attach_prepacked_gives_the_layer_its_buffers(tmp_path):
    from liquidgemm_b200.vllm_plugin import attach_prepacked
    C.save_prepacked(str(tmp_path), [("proj", _layer(256, 128, 5))])
    entry = C.load_prepacked(str(tmp_path))["proj"]
    layer = torch.nn.Linear(128, 256, bias=False)
    attach_prepacked(layer, entry)
    assert layer.lq_enabled and (layer.lq_N, layer.lq_K) == (256, 128) and not hasattr(layer, "weight")
    names = dict(layer.named_buffers())
    assert set(names) == {"lq_s1", "lq_rs", "lq_s_u8", "lq_offset_a"}
    assert torch.equal(names["lq_rs"], entry["rs"])


def test_file_names_from_the_json_cannot_leave_the_directory(tmp_path):
    C.save_prepacked(str(tmp_path), [("a", _layer(128, 128, 6))])
    cfgp = os.path.join(str(tmp_path), C.CONFIG_NAME)
    cfg = json.load(open(cfgp))
    for bad in ("../00000.lqq", "/etc/passwd", "sub/00000.lqq", "00000.bin"):
        cfg["layers"][0]["file"] = bad
        json.dump(cfg, open(cfgp, "w"))
        with pytest.raises(ValueError):
            C.load_prepacked(str(tmp_path))


def test_blob_layout_version_is_checked(tmp_path):
    C.save_prepacked(str(tmp_path), [("a", _layer(128, 128, 7))])
    cfgp = os.path.join(str(tmp_path), C.CONFIG_NAME)
    cfg = json.load(open(cfgp))
    assert cfg["blob_layout"] == C.BLOB_LAYOUT and cfg["tile_bytes"] == C.TILE_BYTES
    cfg["blob_layout"] = C.BLOB_LAYOUT + 1
    json.dump(cfg, open(cfgp, "w"))
    with pytest.raises(ValueError):
        C.read_config(str(tmp_path))
