"""Serialisation of the compressed cache: one self-describing byte blob per layer or per cache.

The reference keeps compressed data only inside a process; a serving stack needs the step after
encode -- move a sequence's compressed KV to host memory or disk (prefix-cache reuse, offload) and
bring it back.  The blob holds exactly what a decode step reads: the used prefix of every
sequence's K and V stream, the block tables, the quantisation parameters, the in-block token order
if blocks were reordered, and (for a cache) the uncompressed residual.  Only bytes move; nothing is
re-encoded.

Layout: b"PKVC" | u32 version | u32 header_len | header (UTF-8 JSON) | payload.  The header lists
every array with dtype, shape and byte offset into the payload (each 16-byte aligned).
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from . import ops

MAGIC, VERSION = b"PKVC", 1
_DTYPES = {"uint8": torch.uint8, "int32": torch.int32, "float16": torch.float16, "bfloat16": torch.bfloat16}
_LAYER_INTS = ("n_comp", "kv_heads", "cbk", "cbv", "bits_k", "bits_v", "k_mode")


def _pack(arrays: Dict[str, torch.Tensor], meta: dict) -> bytes:
    entries, chunks, off = {}, [], 0
    for name, t in arrays.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        entries[name] = {"dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape), "offset": off, "nbytes": len(raw)}
        pad = (-len(raw)) % 16
        chunks.append(raw + b"\0" * pad)
        off += len(raw) + pad
    header = json.dumps({"meta": meta, "arrays": entries}).encode()
    header += b" " * ((-(12 + len(header))) % 16)
    return MAGIC + struct.pack("<II", VERSION, len(header)) + header + b"".join(chunks)


def _unpack(blob: bytes, device) -> Tuple[dict, Dict[str, torch.Tensor]]:
    if len(blob) < 12 or blob[:4] != MAGIC:
        raise ValueError("not a PackKV cache blob")
    version, hlen = struct.unpack("<II", blob[4:12])
    if version != VERSION:
        raise ValueError(f"unsupported blob version {version}")
    if 12 + hlen > len(blob):
        raise ValueError("truncated blob")
    head = json.loads(blob[12:12 + hlen].decode())
    base = 12 + hlen
    arrays = {}
    for name, e in head["arrays"].items():
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"unknown dtype {e['dtype']} for {name}")
        lo, hi = base + e["offset"], base + e["offset"] + e["nbytes"]
        if hi > len(blob):
            raise ValueError("truncated blob")
        dt = _DTYPES[e["dtype"]]
        raw = torch.from_numpy(np.frombuffer(blob, dtype=np.uint8, count=e["nbytes"], offset=lo).copy())
        arrays[name] = (raw.view(dt) if e["nbytes"] else torch.empty(0, dtype=dt)).reshape(e["shape"]).to(device)
    return head["meta"], arrays


def _layer_arrays(layer: ops.CompressedLayer, prefix: str = "") -> Tuple[Dict[str, torch.Tensor], dict]:
    kb, vb = layer.k_bytes.cpu(), layer.v_bytes.cpu()
    k_used = (int(kb.max().item()) + 15) // 16 * 16 if kb.numel() else 0
    v_used = (int(vb.max().item()) + 15) // 16 * 16 if vb.numel() else 0
    nk = (layer.n_comp // layer.cbk) * layer.kv_heads
    nv = (layer.n_comp // layer.cbv) * 2 * layer.kv_heads
    channel = layer.k_mode == ops.K_CHANNEL
    arrays = {
        "k_stream": layer.k_stream[:, :k_used], "k_info": layer.k_info[:, :nk], "k_bytes": layer.k_bytes,
        "k_scale": layer.k_scale[:, :, : layer.n_comp // layer.cbk] if channel else layer.k_scale[:, : layer.n_comp],
        "k_zero": layer.k_zero[:, :, : layer.n_comp // layer.cbk] if channel else layer.k_zero[:, : layer.n_comp],
        "v_stream": layer.v_stream[:, :v_used], "v_info": layer.v_info[:, :nv], "v_bytes": layer.v_bytes,
        "v_scale": layer.v_scale[:, : layer.n_comp], "v_zero": layer.v_zero[:, : layer.n_comp],
    }
    if layer.order is not None:
        arrays["order"] = layer.order
    meta = {k: int(getattr(layer, k)) for k in _LAYER_INTS}
    meta["high_precision_zero"] = bool(layer.high_precision_zero)
    return {prefix + k: v for k, v in arrays.items()}, meta


def _layer_from(meta: dict, arrays: Dict[str, torch.Tensor], prefix: str = "") -> ops.CompressedLayer:
    g = lambda k: arrays[prefix + k]
    k_stream, v_stream = g("k_stream"), g("v_stream")
    # a decode step reads 16-byte chunks and may touch up to 16 bytes past a block: keep a tail
    pad = lambda s: torch.cat([s, torch.zeros(s.shape[0], 32, dtype=torch.uint8, device=s.device)], dim=1).contiguous()
    layer = ops.CompressedLayer(
        k_stream=pad(k_stream), k_info=g("k_info").contiguous(), k_bytes=g("k_bytes"), k_scale=g("k_scale").contiguous(), k_zero=g("k_zero").contiguous(),
        v_stream=pad(v_stream), v_info=g("v_info").contiguous(), v_bytes=g("v_bytes"), v_scale=g("v_scale").contiguous(), v_zero=g("v_zero").contiguous(),
        order=arrays.get(prefix + "order"), high_precision_zero=bool(meta["high_precision_zero"]), **{k: int(meta[k]) for k in _LAYER_INTS})
    # the kernels index the arrays from the metadata: a blob whose metadata and arrays disagree is rejected here
    if layer.bits_k not in (2, 3, 4) or layer.bits_v not in (2, 3, 4) or layer.k_mode not in (ops.K_CHANNEL, ops.K_TOKEN):
        raise ValueError("bad layer metadata")
    ops._check_layer_shapes(layer, int(layer.k_stream.shape[0]))
    return layer


def dumps_layer(layer: ops.CompressedLayer) -> bytes:
    """Compressed layer -> bytes (synchronises: the used stream lengths are read back)."""
    arrays, meta = _layer_arrays(layer)
    return _pack(arrays, {"kind": "layer", "layer": meta})


def loads_layer(blob: bytes, device="cuda") -> ops.CompressedLayer:
    meta, arrays = _unpack(blob, device)
    if meta.get("kind") != "layer":
        raise ValueError("blob does not hold a compressed layer")
    return _layer_from(meta["layer"], arrays)


def dumps_cache(cache) -> bytes:
    """Every layer of a PackKVCache: compressed store + uncompressed residual + lengths."""
    arrays: Dict[str, torch.Tensor] = {}
    layers: List[Optional[dict]] = []
    cache.flush()                      # a decode step's token that no attend() has written yet
    for i, L in enumerate(cache._layers):
        entry = {"n_res": int(L.n_res), "n_comp": int(L.n_comp), "layer": None}
        if L.k_res is not None:
            arrays[f"L{i}.k_res"], arrays[f"L{i}.v_res"] = L.k_res[:, :, : L.n_res], L.v_res[:, :, : L.n_res]
            entry["res_cap"] = int(L.k_res.shape[2])
        if L.comp is not None and L.n_comp:
            a, m = _layer_arrays(L.comp, f"L{i}.")
            arrays.update(a)
            entry["layer"] = m
        layers.append(entry)
    meta = {"kind": "cache", "batch_size": cache.batch_size, "head_num": cache.head_num, "head_dim": cache.head_dim, "layers": layers}
    return _pack(arrays, meta)


def loads_cache(blob: bytes, device="cuda", **cache_kwargs):
    """Rebuilds a PackKVCache (PackKVCacheConfigStatic.config must describe the same quantisation)."""
    from .cache import PackKVCache
    meta, arrays = _unpack(blob, device)
    if meta.get("kind") != "cache":
        raise ValueError("blob does not hold a cache")
    cache = PackKVCache(meta["batch_size"], meta["head_num"], meta["head_dim"], len(meta["layers"]), **cache_kwargs)
    for i, entry in enumerate(meta["layers"]):
        L = cache._layers[i]
        L.n_res, L.n_comp = entry["n_res"], entry["n_comp"]
        if f"L{i}.k_res" in arrays:
            k, v = arrays[f"L{i}.k_res"], arrays[f"L{i}.v_res"]
            cap = max(entry.get("res_cap", k.shape[2]), k.shape[2])
            L.k_res = torch.empty(k.shape[0], k.shape[1], cap, k.shape[3], dtype=k.dtype, device=k.device)
            L.v_res = torch.empty_like(L.k_res)
            L.k_res[:, :, : k.shape[2]], L.v_res[:, :, : k.shape[2]] = k, v
        if entry["layer"] is not None:
            L.comp = _layer_from(entry["layer"], arrays, f"L{i}.")
            L.capacity = L.comp.n_comp          # exactly full: the next append grows the store
    return cache
