"""KV-cache classes with the reference's names and call contract
(models/cache/packkv_cache.py:22-38, models/cache/packkv_quant.py:9-130), backed by the
compressed store instead of a quantise->dequantise simulation.

    PackKVCacheConfigStatic.config = PackKVCacheConfig(...)
    cache = PackKVCache(batch_size, head_num, head_dim, layer_num)
    k_all, v_all = cache.update(key_states, value_states, layer_idx, {"cos": cos, "sin": sin})
    out = cache.attend(query_states, layer_idx)          # fused decompress-attention (decode)

`update` applies RoPE to K inside the cache, appends to the uncompressed residual, and moves whole
token blocks into the packed streams by the reference's cut rule (utils/compute.py:54-67): with
block 64 and buffer 192 the residual holds 128..191 tokens and every 64th decode step packs one
block.  For prefill (more than one new token), for `materialize=True` and when quantisation is
disabled it returns dense K/V exactly like the reference (dequantised history + residual); on a
decode step with `materialize=False` it returns (None, None) and `attend` computes the attention
straight from the packed streams.

With the installed transformers (5.x) the attention modules rotate K themselves and call
`update(key_states, value_states, layer_idx)` without sin/cos: then no RoPE is applied here.
`decode_handles=True` makes a decode step return a pair of `PackKVHandle`s instead of
(None, None); the attention function registered by `packkv_b200.hf` turns them into a call of
`attend`.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import encode, ops
from .config import PackKVCacheConfig, QuantMode, RepackMethod

try:  # the installed transformers' Cache needs constructor arguments the reference never passed
    from transformers import Cache as _HFCache
except Exception:  # pragma: no cover - transformers is optional
    _HFCache = object


class PackKVCacheConfigStatic:
    """Process-wide configuration slot, as in the reference (packkv_quant.py:9-11)."""
    config: Optional[PackKVCacheConfig] = None
    extract_cache = None


def bits_for_rel(rel: float) -> int:
    """Bit width the quantiser's codes need: it produces at most round(1/rel) + 2 levels."""
    return max(2, math.ceil(math.log2(math.floor(1.0 / rel + 1e-6) + 2)))


def compress_block_count(length: int, block: int, recent: int) -> int:
    """Whole blocks that leave a residual of `length` tokens (utils/compute.py:60-62)."""
    return max(0, (length + block - length % block - recent) // block)


class PackKVHandle:
    """Stands in for the K (or V) tensor of a decode step: names the cache and the layer."""
    __slots__ = ("cache", "layer_idx")

    def __init__(self, cache: "PackKVCache", layer_idx: int):
        self.cache, self.layer_idx = cache, layer_idx


class _Layer:
    def __init__(self):
        self.comp: Optional[ops.CompressedLayer] = None
        self.capacity = 0          # tokens the compressed store has room for
        self.k_res: Optional[torch.Tensor] = None
        self.v_res: Optional[torch.Tensor] = None
        self.n_res = 0
        self.n_comp = 0
        self.pending = None        # (k_new, v_new, cos, sin) of a decode step whose token the next attend() writes into row n_res - 1


class PackKVCache(_HFCache):
    def __init__(self, batch_size, head_num, head_dim, layer_num, materialize: bool = False, decode_handles: bool = False):
        if _HFCache is not object:
            try:
                super().__init__(layers=[])
            except TypeError:
                try:
                    super().__init__()
                except Exception:
                    pass
        self.batch_size = batch_size
        self.head_num = head_num          # the models pass num_attention_heads; KV heads come from the tensors
        self.head_dim = head_dim
        self.materialize = materialize
        self.decode_handles = decode_handles
        self._layers: List[_Layer] = [_Layer() for _ in range(layer_num)]
        self.flags: Optional[torch.Tensor] = None
        self._scratch: Optional[torch.Tensor] = None   # hand-over area of the attention's two-launch form

    # ---------------------------------------------------------------------------------------------
    @staticmethod
    def _config() -> PackKVCacheConfig:
        cfg = PackKVCacheConfigStatic.config
        if cfg is None:
            raise ValueError("TComCacheConfigStatic.config is not set. Please set it before using TComCache.")
        return cfg

    def check_flags(self):
        """Reads the device status word (synchronises) and raises if a kernel reported a condition that makes
        the cache's contents or an attention result wrong.  update() and attend() are asynchronous and do not
        call this; compressed_bytes() does, and callers should at points where they synchronise anyway."""
        f = int(self.flags.item()) if self.flags is not None else 0
        if f:
            raise RuntimeError(f"PackKV device status flags set: {f} (1=stream overflow, 2=code range, 4=bad stream, "
                               "8=wait timed out, 16=zero-point outside the exact range of the attention kernel)")

    _check_flags = check_flags

    def _ensure_store(self, L: _Layer, kv_heads: int, need_tokens: int, dtype, device, cfg: PackKVCacheConfig):
        if L.comp is not None and L.capacity >= need_tokens:
            return
        block = cfg.block_size
        cap = max(need_tokens, 2 * L.capacity, 16 * block)
        cap = (cap + 127) // 128 * 128
        bits_k, bits_v = bits_for_rel(cfg.k_quant_scale_rel), bits_for_rel(cfg.v_quant_scale_rel)
        k_mode = cfg.quant_method.value[0]
        B = self.batch_size
        new = ops.CompressedLayer(
            k_stream=torch.zeros(B, encode.stream_capacity("k", cap, kv_heads, block, bits_k), dtype=torch.uint8, device=device),
            k_info=torch.zeros(B, (cap // block) * kv_heads, 2, dtype=torch.int32, device=device),
            k_bytes=torch.zeros(B, dtype=torch.int32, device=device),
            k_scale=torch.zeros((B, kv_heads, cap // block, 128) if k_mode == QuantMode.ChannelQuant else (B, cap), dtype=dtype, device=device),
            k_zero=torch.zeros((B, kv_heads, cap // block, 128) if k_mode == QuantMode.ChannelQuant else (B, cap), dtype=dtype, device=device),
            v_stream=torch.zeros(B, encode.stream_capacity("v", cap, kv_heads, block, bits_v), dtype=torch.uint8, device=device),
            v_info=torch.zeros(B, (cap // block) * 2 * kv_heads, 2, dtype=torch.int32, device=device),
            v_bytes=torch.zeros(B, dtype=torch.int32, device=device),
            v_scale=torch.zeros(B, cap, dtype=dtype, device=device), v_zero=torch.zeros(B, cap, dtype=dtype, device=device),
            n_comp=0, kv_heads=kv_heads, cbk=block, cbv=block, bits_k=bits_k, bits_v=bits_v,
            k_mode=ops.K_CHANNEL if k_mode == QuantMode.ChannelQuant else ops.K_TOKEN,
            high_precision_zero=bool(cfg.high_precision_zero_point))
        old = L.comp
        if old is not None:   # grow: copy the used prefix of every buffer
            new.k_stream[:, : old.k_stream.shape[1]] = old.k_stream
            new.v_stream[:, : old.v_stream.shape[1]] = old.v_stream
            new.k_info[:, : old.k_info.shape[1]] = old.k_info
            new.v_info[:, : old.v_info.shape[1]] = old.v_info
            new.k_bytes.copy_(old.k_bytes)
            new.v_bytes.copy_(old.v_bytes)
            if new.k_mode == ops.K_CHANNEL:
                new.k_scale[:, :, : old.k_scale.shape[2]] = old.k_scale
                new.k_zero[:, :, : old.k_zero.shape[2]] = old.k_zero
            else:
                new.k_scale[:, : old.k_scale.shape[1]] = old.k_scale
                new.k_zero[:, : old.k_zero.shape[1]] = old.k_zero
            new.v_scale[:, : old.v_scale.shape[1]] = old.v_scale
            new.v_zero[:, : old.v_zero.shape[1]] = old.v_zero
            new.n_comp = old.n_comp
            new.order = old.order
        L.comp, L.capacity = new, cap

    def _compress(self, L: _Layer, k: torch.Tensor, v: torch.Tensor, cfg: PackKVCacheConfig):
        """Quantises and packs k, v (B, H, n*block, 128) behind the tokens already stored."""
        B, H, n, _ = k.shape
        self._ensure_store(L, H, L.n_comp + n, k.dtype, k.device, cfg)
        C, block = L.comp, cfg.block_size
        if self.flags is None:
            self.flags = ops.new_flags(k.device)
        if cfg.repack_method in (RepackMethod.MEDIAN, RepackMethod.GREEDY):
            # quantise, reorder the tokens of each new block (median of the V codes, or greedy packs), pack
            kq = ops.quantize(k, block, cfg.k_quant_scale_rel, C.k_mode, bits=C.bits_k, high_precision_zero=C.high_precision_zero,
                              flags=self.flags, scale=C.k_scale, zero=C.k_zero, first_token=L.n_comp)
            vq = ops.quantize(v, block, cfg.v_quant_scale_rel, ops.K_TOKEN, bits=C.bits_v, high_precision_zero=C.high_precision_zero,
                              flags=self.flags, scale=C.v_scale, zero=C.v_zero, first_token=L.n_comp)
            order = (ops.median_order(vq.codes, H, block) if cfg.repack_method == RepackMethod.MEDIAN
                     else ops.greedy_order(kq.codes, vq.codes, H, block, cfg.pack_size))
            C.v_scale = ops.gather_params(C.v_scale, order, block, n, first=L.n_comp)
            C.v_zero = ops.gather_params(C.v_zero, order, block, n, first=L.n_comp)
            if C.k_mode == ops.K_TOKEN:
                C.k_scale = ops.gather_params(C.k_scale, order, block, n, first=L.n_comp)
                C.k_zero = ops.gather_params(C.k_zero, order, block, n, first=L.n_comp)
            ops.encode_codes("k", ops.gather_rows(kq.codes, order, block), C.cbk, C.bits_k, stream=C.k_stream, info=C.k_info,
                             stream_bytes=C.k_bytes, flags=self.flags, first_cb=L.n_comp // C.cbk)
            ops.encode_codes("v", ops.gather_rows(vq.codes, order, block), C.cbv, C.bits_v, stream=C.v_stream, info=C.v_info,
                             stream_bytes=C.v_bytes, flags=self.flags, first_cb=L.n_comp // C.cbv)
            C.order = order if C.order is None else torch.cat([C.order, order], dim=1)
        else:
            scratch = torch.empty(max(16, B * n * H * 128), dtype=torch.uint8, device=k.device)
            ops.encode_tensor("k", k, block, cfg.k_quant_scale_rel, C.k_mode, C.bits_k, C.cbk, scale=C.k_scale, zero=C.k_zero,
                              stream=C.k_stream, info=C.k_info, stream_bytes=C.k_bytes, flags=self.flags, first_token=L.n_comp,
                              high_precision_zero=C.high_precision_zero, scratch=scratch)
            ops.encode_tensor("v", v, block, cfg.v_quant_scale_rel, ops.K_TOKEN, C.bits_v, C.cbv, scale=C.v_scale, zero=C.v_zero,
                              stream=C.v_stream, info=C.v_info, stream_bytes=C.v_bytes, flags=self.flags, first_token=L.n_comp,
                              high_precision_zero=C.high_precision_zero, scratch=scratch)
        L.n_comp += n
        C.n_comp = L.n_comp

    # ---------------------------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None, **_unused) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        cfg = self._config()
        if PackKVCacheConfigStatic.extract_cache is not None:
            assert not cfg.enable_quant, "Disable quant to enable cache collect."
        L = self._layers[layer_idx]
        self._flush(L)
        B, H, T, D = key_states.shape
        if D != 128 and (D > 128 or D < 64 or D % 8):
            raise RuntimeError("not supported")   # streams are built from 128-channel blocks; 64..120 are padded, see _widen
        if cfg.enable_quant and cfg.block_size not in (64, 128):
            # the codec packs 32-token blocks too, but the attention kernel reads 64- and 128-token blocks only:
            # refuse here, not at the first attend()
            raise RuntimeError("not supported: PackKVCache needs block_size 64 or 128")
        # the reference's models pass K before RoPE together with sin/cos; the installed transformers rotates K itself
        cos, sin = (cache_kwargs["cos"], cache_kwargs["sin"]) if cache_kwargs is not None and "cos" in cache_kwargs and "sin" in cache_kwargs else (None, None)
        if D != 128 and cfg.enable_quant:
            if cos is not None:
                key_states, cos, sin = ops.rope(key_states, cos, sin), None, None
            key_states, value_states = self._widen(key_states), self._widen(value_states)
            D = 128
        if cfg.enable_quant and L.k_res is not None:
            total = L.n_res + T
            if compress_block_count(total, cfg.block_size, cfg.buffer_size) == 0:
                # the common decode step: rotate K and copy V straight into the residual.  With one new token and
                # the fused attention to follow, the attention launch does it itself (attend() below); otherwise one launch
                if T == 1 and not self.materialize and key_states.dtype in (torch.float16, torch.bfloat16):
                    if cos is not None:
                        cos, sin = cos.to(key_states.dtype).contiguous(), sin.to(key_states.dtype).contiguous()
                    L.pending = (key_states, value_states, cos, sin)
                else:
                    ops.append_residual(key_states, value_states, L.k_res, L.v_res, L.n_res, cos, sin)
                L.n_res = total
                return self._step_result(layer_idx, T)
        k_new = ops.rope(key_states, cos, sin) if cos is not None else key_states.contiguous()
        v_new = value_states
        if not cfg.enable_quant:
            L.k_res = k_new if L.k_res is None else torch.cat([L.k_res[:, :, : L.n_res], k_new], dim=2)
            L.v_res = v_new.clone() if L.v_res is None else torch.cat([L.v_res[:, :, : L.n_res], v_new], dim=2)
            L.n_res += T
            ex = PackKVCacheConfigStatic.extract_cache
            if ex is not None:
                ex.key_caches.setdefault(0, {})[layer_idx - 1] = L.k_res
                ex.value_caches.setdefault(0, {})[layer_idx - 1] = L.v_res
            return L.k_res, L.v_res

        block, recent = cfg.block_size, cfg.buffer_size
        total = L.n_res + T
        n_c = compress_block_count(total, block, recent) * block
        res_cap = recent + block
        if L.k_res is None:
            L.k_res = torch.empty(B, H, res_cap, D, dtype=k_new.dtype, device=k_new.device)
            L.v_res = torch.empty(B, H, res_cap, D, dtype=k_new.dtype, device=k_new.device)
        if n_c == 0:
            L.k_res[:, :, L.n_res: total] = k_new
            L.v_res[:, :, L.n_res: total] = v_new
            L.n_res = total
        else:
            if L.n_res:
                k_all = torch.cat([L.k_res[:, :, : L.n_res], k_new], dim=2)
                v_all = torch.cat([L.v_res[:, :, : L.n_res], v_new], dim=2)
            else:
                k_all, v_all = k_new, v_new
            self._compress(L, k_all[:, :, :n_c], v_all[:, :, :n_c], cfg)
            L.n_res = total - n_c
            L.k_res[:, :, : L.n_res] = k_all[:, :, n_c:]
            L.v_res[:, :, : L.n_res] = v_all[:, :, n_c:]
        return self._step_result(layer_idx, T)

    def _flush(self, L: "_Layer") -> None:
        """Writes a decode step's token that no attend() has consumed into the residual (one launch)."""
        if L.pending is not None:
            k_new, v_new, cos, sin = L.pending
            L.pending = None
            ops.append_residual(k_new, v_new, L.k_res, L.v_res, L.n_res - 1, cos, sin)

    def flush(self) -> None:
        """Makes the residual buffers of every layer complete (call before reading them from outside)."""
        for L in self._layers:
            self._flush(L)

    @staticmethod
    def _widen(x: torch.Tensor) -> torch.Tensor:
        """(B, H, T, D) with 64 <= D < 128 -> (B, H, T, 128): the tail repeats the first 128 - D channels.  The
        streams are built from 128-channel blocks; with copies in the tail the per-channel K parameters of the real
        channels and the per-token minima / maxima of V (and token-mode K) are unchanged, so codes and parameters
        of the real channels are exactly the reference's for head_dim D.  attend() pads q with zeros, so the copies
        add nothing to the scores, and drops the tail of the output."""
        return torch.cat([x, x[..., : 128 - x.shape[-1]]], dim=-1)

    def _step_result(self, layer_idx: int, T: int):
        if T > 1 or self.materialize:
            return self.dense(layer_idx)
        if self.decode_handles:
            return PackKVHandle(self, layer_idx), PackKVHandle(self, layer_idx)
        return None, None

    def dense(self, layer_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dequantised history + residual, (B, H, S, 128): what the reference's update returns."""
        L = self._layers[layer_idx]
        self._flush(L)
        D = self.head_dim if self.head_dim < 128 else 128
        k_res, v_res = L.k_res[:, :, : L.n_res, :D], L.v_res[:, :, : L.n_res, :D]
        if L.n_comp == 0:
            return k_res.clone(), v_res.clone()
        C, cfg = L.comp, self._config()
        H = C.kv_heads
        kc, _ = ops.decode_codes("k", C.k_stream, C.k_info, L.n_comp, H * 128, C.cbk, C.bits_k, flags=self.flags)
        vc, _ = ops.decode_codes("v", C.v_stream, C.v_info, L.n_comp, H * 128, C.cbv, C.bits_v, flags=self.flags)
        kd = ops.dequantize(kc, C.k_scale, C.k_zero, H, cfg.block_size, C.k_mode, high_precision_zero=C.high_precision_zero)
        vd = ops.dequantize(vc, C.v_scale, C.v_zero, H, cfg.block_size, ops.K_TOKEN, high_precision_zero=C.high_precision_zero)
        if C.order is not None:   # undo the in-block reordering: original position of every stored row
            block = cfg.block_size
            pos = (C.order.to(torch.int64) + torch.arange(L.n_comp // block, device=kd.device).view(1, -1, 1) * block).reshape(kd.shape[0], -1)
            inv = torch.empty_like(pos)
            inv.scatter_(1, pos, torch.arange(L.n_comp, device=kd.device).expand_as(pos))
            idx = inv.view(kd.shape[0], 1, L.n_comp, 1).expand_as(kd)
            kd, vd = torch.gather(kd, 2, idx), torch.gather(vd, 2, idx)
        return torch.cat([kd[..., :D], k_res], dim=2), torch.cat([vd[..., :D], v_res], dim=2)

    def attend(self, query_states: torch.Tensor, layer_idx: int, scaling: Optional[float] = None) -> torch.Tensor:
        """Decode attention for one new token: query_states (B, Hq, 1, 128) after RoPE ->
        (B, 1, Hq, 128), the layout the reference's eager attention returns (llama.py:210-212)."""
        L = self._layers[layer_idx]
        B, Hq, T, D = query_states.shape
        if T != 1:
            raise ValueError("attend handles one query token per sequence; use dense() for prefill")
        if self.flags is None:
            self.flags = ops.new_flags(query_states.device)
        q = query_states.reshape(B, Hq, D)
        if D != 128:
            if scaling is None:
                scaling = D ** -0.5
            q = torch.nn.functional.pad(q, (0, 128 - D))       # zeros: the copied channels of K add nothing
        q = q.contiguous()
        kv_heads = L.comp.kv_heads if L.comp is not None else L.k_res.shape[1]
        pending, L.pending = L.pending, None
        if self._scratch is None and B * kv_heads <= 64:
            # few (sequence, KV head) pairs: let the library split each over several clusters (all layers share the
            # area: their launches are ordered on one stream)
            self._scratch = ops.new_attention_scratch(q.device)
        out = ops.decode_attention(q, L.comp if L.n_comp else None, L.k_res, L.v_res, L.n_res, scaling=scaling,
                                   flags=self.flags, kv_heads=kv_heads, append=pending, scratch=self._scratch)
        return out.view(B, 1, Hq, 128)[..., :D]

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        self._config()
        L = self._layers[0 if layer_idx is None else layer_idx]
        return L.n_comp + L.n_res

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0) -> Tuple[int, int]:
        """(kv_length, kv_offset) of the mask transformers builds before this layer's update."""
        return self.get_seq_length(layer_idx) + int(query_length), 0

    def compressed_bytes(self) -> int:
        """Bytes of packed streams held by all layers (synchronises, and checks the device status word)."""
        self.check_flags()
        n = 0
        for L in self._layers:
            if L.comp is not None:
                n += int(L.comp.k_bytes.sum().item()) + int(L.comp.v_bytes.sum().item())
        return n


# the reference keeps the implementation behind a second class name (packkv_quant.py:30)
PackKVCachePytorchQuant = PackKVCache
