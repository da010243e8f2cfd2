"""Minimal GGUF v3 writer for the tests: the container format the reference's converter
produces (tools/convert_omni.py uses the `gguf` package; this restates the published layout).

Header: magic "GGUF", version 3, tensor count, key/value count (little endian); key/value
pairs (string key, u32 value type, value); tensor infos (string name, u32 rank, u64 extents with
ne[0] the row length, u32 element type, u64 offset into the data section); padding to
`general.alignment`; tensor data, each tensor aligned.
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np
import torch

F32, F16, BF16 = 0, 1, 30
T_U32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_I32 = 4, 6, 7, 8, 9, 5


def _s(b: str | bytes) -> bytes:
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def _kv(key, value) -> bytes:
    if isinstance(value, bool):
        return _s(key) + struct.pack("<IB", T_BOOL, int(value))
    if isinstance(value, float):
        return _s(key) + struct.pack("<If", T_F32, value)
    if isinstance(value, int):
        return _s(key) + struct.pack("<II", T_U32, value)
    if isinstance(value, str):
        return _s(key) + struct.pack("<I", T_STRING) + _s(value)
    if isinstance(value, (list, tuple)) and all(isinstance(v, str) for v in value):
        return _s(key) + struct.pack("<IIQ", T_ARRAY, T_STRING, len(value)) + b"".join(_s(v) for v in value)
    if isinstance(value, (list, tuple)):
        return _s(key) + struct.pack("<IIQ", T_ARRAY, T_I32, len(value)) + struct.pack(f"<{len(value)}i", *value)
    raise TypeError(type(value))


def _bytes(t) -> bytes:
    if isinstance(t, torch.Tensor):
        t = t.contiguous()
        return (t.view(torch.uint8) if t.dtype != torch.uint8 else t).numpy().tobytes()
    return np.ascontiguousarray(t).tobytes()


def write_gguf(path: Path, kv: dict, tensors: dict, alignment: int = 32, version: int = 3, magic: bytes = b"GGUF",
               misalign: str | None = None, truncate: int = 0) -> None:
    """tensors: name -> (ggml type, tensor); the tensor's shape is [.., rows, row length] and is
    written reversed, as GGUF stores extents."""
    kv = dict(kv)
    kv.setdefault("general.alignment", alignment)
    head = magic + struct.pack("<IQQ", version, len(tensors), len(kv)) + b"".join(_kv(k, v) for k, v in kv.items())
    infos, blobs, off = b"", [], 0
    for name, (ty, t) in tensors.items():
        raw = _bytes(t)
        shape = tuple(t.shape)[::-1]
        o = off + (4 if misalign == name else 0)
        infos += _s(name) + struct.pack("<I", len(shape)) + struct.pack(f"<{len(shape)}Q", *shape) + struct.pack("<IQ", ty, o)
        blobs.append((o, raw))
        off = (o + len(raw) + alignment - 1) // alignment * alignment
    body = head + infos
    body += b"\0" * ((-len(body)) % alignment)
    with open(path, "wb") as f:
        f.write(body)
        base = len(body)
        for o, raw in blobs:
            f.seek(base + o)
            f.write(raw)
        end = base + off
        f.truncate(max(0, end - truncate))


def omni_layers(weights_per_layer, norms, H, ffn, E):
    """The tensors of the MoE block, named as the reference's engine binds them (clef.c:232-246)."""
    out = {}
    for l, ((router, gate_up, down), norm) in enumerate(zip(weights_per_layer, norms)):
        assert tuple(router.shape) == (E, H) and tuple(gate_up.shape) == (E, 2 * ffn, H) and tuple(down.shape) == (E, H, ffn)
        out[f"blk.{l}.ffn_norm.weight"] = (F32, norm)
        out[f"blk.{l}.ffn_router.weight"] = (BF16, router)
        out[f"blk.{l}.ffn_gate_up_exps.weight"] = (BF16, gate_up)
        out[f"blk.{l}.ffn_down_exps.weight"] = (BF16, down)
    return out


def omni_kv(H, ffn, E, used, n_layer, eps=1e-6):
    """The metadata keys that pin the block's geometry (clef.c:27-36, 55, 76-79), plus a few of
    other types so that the reader's value skipping is exercised."""
    return {"general.architecture": "clef", "clef.block_count": n_layer, "clef.embedding_length": H,
            "clef.feed_forward_length": ffn, "clef.moe.expert_count": E, "clef.moe.expert_used_count": used,
            "clef.moe.normalize_topk": True, "clef.attention.layer_norm_rms_epsilon": eps,
            "tokenizer.tokens": ["a", "bc", ""], "clef.rope.mrope_section": [24, 20, 20]}
