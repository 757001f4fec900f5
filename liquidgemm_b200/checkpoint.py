"""Serialised prepacked LQQ layers: quantise and prepack once, load the tile blobs directly afterwards.

The reference has no on-disk format: every start-up re-quantises the bf16 checkpoint
(liquidgemm/vllm_plugin.py:136-172) and its config hooks are stubs (``get_config_filenames`` returns
``[]``, liquidgemm/vllm_plugin.py:92-99).  This module defines one:

``<dir>/liquidgemm_config.json``   format version, blob layout version, group size, the layer table (name, N, K,
                                   file, sha256)
``<dir>/<index>.lqq``              one file per layer: ``torch.save`` of ``{"rs", "s1", "s_u8", "offset_a"}``
                                   as CPU tensors (``rs`` is the tile blob the kernels read)

``load_prepacked`` checks version, shapes, blob sizes and (optionally) the hashes, so a truncated or
foreign file fails loudly instead of producing wrong logits.
"""

from __future__ import annotations

import hashlib
import json
import os
import re
from typing import Dict, Iterable, Tuple

import torch

FORMAT = "liquidgemm-b200-prepacked"
VERSION = 1
CONFIG_NAME = "liquidgemm_config.json"
TILE_BYTES = 8704
# Version of the tile blob itself (4 x [128 rows][16 B] interleaved nibbles + [128][step0, off0, step1, off1]
# per 128 x 128 tile); a change of that layout must bump it so that old directories are refused.
BLOB_LAYOUT = 1
_FILE_RE = re.compile(r"^[0-9]{5}\.lqq$")


def blob_bytes(N: int, K: int) -> int:
    """Size of the tile blob of an [N, K] layer (128 x 128 tiles of 8704 bytes, rows padded)."""
    return ((N + 127) // 128) * (K // 128) * TILE_BYTES


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def save_prepacked(directory: str, layers: Iterable[Tuple[str, dict]], group_size: int = 64) -> str:
    """Write ``layers`` (name, {"rs", "s1", "s_u8", "offset_a", "N", "K"}) to ``directory``; returns the
    path of the config file."""
    os.makedirs(directory, exist_ok=True)
    table = []
    for i, (name, L) in enumerate(layers):
        N, K = int(L["N"]), int(L["K"])
        rs = L["rs"].detach().reshape(-1).cpu().contiguous()
        if rs.dtype != torch.uint8 or rs.numel() != blob_bytes(N, K):
            raise ValueError(f"{name}: tile blob has {rs.numel()} bytes, expected {blob_bytes(N, K)} for {N}x{K}")
        payload = {"rs": rs, "s1": L["s1"].detach().float().cpu().contiguous(),
                   "s_u8": L["s_u8"].detach().cpu().contiguous(), "offset_a": L["offset_a"].detach().cpu().contiguous()}
        if payload["s1"].numel() != N or payload["s_u8"].numel() != N * (K // group_size):
            raise ValueError(f"{name}: scale tensors do not match {N}x{K} with group size {group_size}")
        fname = f"{i:05d}.lqq"
        path = os.path.join(directory, fname)
        torch.save(payload, path)
        table.append({"name": name, "N": N, "K": K, "file": fname, "sha256": _sha256(path)})
    cfg = {"format": FORMAT, "version": VERSION, "blob_layout": BLOB_LAYOUT, "tile_bytes": TILE_BYTES,
           "quant_method": "liquidgemm", "group_size": int(group_size), "w4": True, "layers": table}
    cfg_path = os.path.join(directory, CONFIG_NAME)
    with open(cfg_path, "w") as f:
        json.dump(cfg, f, indent=1)
    return cfg_path


def read_config(directory: str) -> dict:
    with open(os.path.join(directory, CONFIG_NAME)) as f:
        cfg = json.load(f)
    if cfg.get("format") != FORMAT:
        raise ValueError(f"{directory}: not a {FORMAT} directory")
    if int(cfg.get("version", -1)) != VERSION:
        raise ValueError(f"{directory}: format version {cfg.get('version')} is not supported (expected {VERSION})")
    if int(cfg.get("blob_layout", -1)) != BLOB_LAYOUT or int(cfg.get("tile_bytes", -1)) != TILE_BYTES:
        raise ValueError(f"{directory}: tile blob layout {cfg.get('blob_layout')} / {cfg.get('tile_bytes')} bytes per "
                         f"tile is not the one this library reads ({BLOB_LAYOUT} / {TILE_BYTES})")
    for ent in cfg.get("layers", []):
        # the file name comes from the json: it must be a plain NNNNN.lqq inside the directory
        if not isinstance(ent.get("file"), str) or not _FILE_RE.match(ent["file"]):
            raise ValueError(f"{directory}: layer {ent.get('name')!r} names the file {ent.get('file')!r}; "
                             "expected NNNNN.lqq inside the directory")
    return cfg


def load_prepacked(directory: str, device="cpu", verify_hashes: bool = True) -> Dict[str, dict]:
    """Read every layer back as {"rs", "s1", "s_u8", "offset_a", "N", "K"} on ``device``."""
    cfg = read_config(directory)
    g = int(cfg["group_size"])
    out = {}
    for ent in cfg["layers"]:
        path = os.path.join(directory, ent["file"])
        if verify_hashes and _sha256(path) != ent["sha256"]:
            raise ValueError(f"{path}: content hash differs from the one recorded in {CONFIG_NAME}")
        t = torch.load(path, map_location="cpu", weights_only=True)
        N, K = int(ent["N"]), int(ent["K"])
        if t["rs"].dtype != torch.uint8 or t["rs"].numel() != blob_bytes(N, K):
            raise ValueError(f"{path}: tile blob size does not match {N}x{K}")
        if t["s1"].numel() != N or t["s_u8"].numel() != N * (K // g) or t["offset_a"].numel() != N * (K // g):
            raise ValueError(f"{path}: scale tensors do not match {N}x{K} with group size {g}")
        out[ent["name"]] = {"rs": t["rs"].to(device), "s1": t["s1"].to(device), "s_u8": t["s_u8"].to(device),
                            "offset_a": t["offset_a"].to(device), "N": N, "K": K}
    return out
