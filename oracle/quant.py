"""CPU restatement of the reference's quantiser, reorder heuristic, cache bookkeeping and
decompress-then-attend path.  TEST INFRASTRUCTURE ONLY (tests, smoke check, CPU baseline).

The reference does this arithmetic with PyTorch ops on fp16/bf16 tensors, so every op
rounds to the tensor dtype; the restatement keeps the same op order and dtype so that codes,
zero-points and scales come out bit-identical on CPU.  Parity status: pinned -- the tests
compare every function here with the reference's own ``utils/compute.py`` imported from the
checkout when it is present, and with committed fixtures made that way.

Reference lines followed:
  quant_ints                  utils/compute.py:84-112   (QUANT_DIM :405-410)
  dequantise                  utils/compute.py:173-178
  cut_tensor                  utils/compute.py:54-67
  median_repacking            utils/compute.py:262-270
  bit_pack (size model)       utils/compute.py:272-297
  apply_rotary_pos_emb_single utils/compute.py:22-43
  codes -> (ctx, hidden) u8   evaluation/evaluation.py:406,596
  eager attention             models/llama.py:177-212
  cache update                models/cache/packkv_quant.py:45-85
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

# reduction dims on the 5-D view (B, H, n_blocks, block, D)
QUANT_DIMS = {"block": (1, 3, 4), "channel": (3,), "token": (1, 4), "vector": (4,)}


def quant_ints(x: torch.Tensor, block: int, rel: float, mode: str, high_precision_zero: bool = False):
    """(B,H,S,D) -> codes (B,H,nb,block,D), zero, scale (keep-dim shapes), all in x.dtype."""
    assert x.shape[2] % block == 0
    t = x.reshape(x.shape[0], x.shape[1], -1, block, x.shape[3])
    lo, hi = t, t
    for d in QUANT_DIMS[mode]:
        lo = lo.min(dim=d, keepdim=True).values
        hi = hi.max(dim=d, keepdim=True).values
    scale = (hi - lo) * rel
    if high_precision_zero:
        return ((t - lo) / scale).round(), lo, scale
    zero = (lo / scale).round()
    return (t / scale).round() - zero, zero, scale


def dequant(codes, zero, scale, high_precision_zero: bool = False):
    """Inverse used by the reference's cache; result (B,H,S,D)."""
    y = codes * scale + zero if high_precision_zero else (codes + zero) * scale
    return y.reshape(y.shape[0], y.shape[1], -1, y.shape[4])


def codes_matrix(codes5: torch.Tensor) -> torch.Tensor:
    """(B,H,nb,block,D) float codes -> (ctx, B*H*D) uint8, the codec's input layout."""
    return codes5.flatten(2, 3).permute(2, 0, 1, 3).flatten(1, 3).contiguous().to(torch.uint8)


def compress_block_count(length: int, block: int, recent: int) -> int:
    """How many whole blocks leave a residual buffer holding `length` tokens."""
    return max(0, (length + block - length % block - recent) // block)


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rope(t, cos, sin):
    """t (B,H,S,D); cos/sin (B,S,D)."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return (t * cos) + (rotate_half(t) * sin)


def median_order(blocks: torch.Tensor) -> torch.Tensor:
    """blocks (n_blocks, block, 2F) codes with K features first, V features second.
    Returns the token order (n_blocks, block) int64: descending lower-median of the V half."""
    f = blocks.shape[2] // 2
    med = torch.median(blocks[:, :, f:], dim=2).values
    return torch.sort(med, dim=1, descending=True).indices


def median_reorder(blocks: torch.Tensor) -> torch.Tensor:
    order = median_order(blocks)
    return torch.gather(blocks, 1, order.unsqueeze(2).expand_as(blocks))


def greedy_order(blocks: torch.Tensor, pack_len: int) -> torch.Tensor:
    """Token order (n_blocks, block) int64 of the reference's greedy_repacking
    (utils/compute.py:210-260), restated with exact integer arithmetic: the seed of a pack is the
    remaining token with the largest cosine to the rounded mean of the remaining tokens (compared
    as dot^2/|x|^2 by cross-multiplication: the mean's norm is common and dots are non-negative),
    every further token is the first remaining one that minimises the pack's bit count
    sum_f bit_length(max_f - min_f).  The reference evaluates the cosine in fp32; both agree unless
    two candidates tie within fp32 rounding."""
    import numpy as np
    x = blocks.to(torch.int64).numpy()
    nb, n, f = x.shape
    order = np.zeros((nb, n), dtype=np.int64)
    bl = np.array([int(v).bit_length() for v in range(256)], dtype=np.int64)
    for b in range(nb):
        rem = list(range(n))
        out = []
        for _ in range(n // pack_len):
            xs = x[b, rem]                                   # (r, f)
            tot, r = xs.sum(axis=0), len(rem)
            q, r2 = tot // r, 2 * (tot % r)
            mean = q + ((r2 > r) | ((r2 == r) & (q % 2 == 1)))
            dots = (xs * mean).sum(axis=1)
            nrm = (xs * xs).sum(axis=1)
            best = 0
            for c in range(1, r):
                d2, n2, bd, bn = int(dots[c]) ** 2, int(nrm[c]), int(dots[best]) ** 2, int(nrm[best])
                gt = False if n2 == 0 else (d2 > 0 if bn == 0 else d2 * bn > bd * n2)
                if gt:
                    best = c
            tok = rem.pop(best)
            out.append(tok)
            lo = x[b, tok].copy()
            hi = lo.copy()
            for _ in range(pack_len - 1):
                if not rem:
                    break
                xs = x[b, rem]
                cost = bl[np.maximum(xs, hi) - np.minimum(xs, lo)].sum(axis=1)
                tok = rem.pop(int(np.argmin(cost)))
                out.append(tok)
                lo, hi = np.minimum(lo, x[b, tok]), np.maximum(hi, x[b, tok])
        order[b] = out
    return torch.from_numpy(order)


def greedy_reorder(blocks: torch.Tensor, pack_len: int) -> torch.Tensor:
    order = greedy_order(blocks, pack_len)
    return torch.gather(blocks, 1, order.unsqueeze(2).expand_as(blocks))


def kv_feature_blocks(k_codes5: torch.Tensor, v_codes5: torch.Tensor) -> torch.Tensor:
    """(B,H,nb,block,D) x2 -> (nb, block, 2*B*H*D), compute.py:336-338."""
    kb = k_codes5.permute(2, 3, 0, 1, 4).flatten(2, 4)
    vb = v_codes5.permute(2, 3, 0, 1, 4).flatten(2, 4)
    return torch.cat([kb, vb], dim=2)


def size_model(blocks: torch.Tensor, pack_len: int) -> Tuple[int, int]:
    """Bytes the size model predicts for the K half and the V half."""
    f = blocks.shape[2] // 2
    b = blocks.flatten(0, 1).to(torch.int64)
    out = []
    for part in (b[:, :f], b[:, f:]):
        packs = part.reshape(-1, pack_len, f)
        raw = math.ceil(math.log2(packs.unique().numel()))
        lo, hi = packs.min(dim=1).values, packs.max(dim=1).values
        bits = torch.ceil(torch.log2((hi - lo + 1).to(torch.float32))).to(torch.int64).sum() * pack_len
        bits = bits + lo.numel() * (raw + math.ceil(math.log2(raw + 1)))
        out.append(int(bits.item()) // 8)
    return out[0], out[1]


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    b, h, s, d = x.shape
    if n_rep == 1:
        return x
    return x[:, :, None].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)


def eager_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: Optional[float] = None):
    """q (B,Hq,T,D), k/v (B,Hkv,S,D) -> (B,T,Hq,D); fp32 softmax, no mask (decode)."""
    g = q.shape[1] // k.shape[1]
    ks, vs = repeat_kv(k, g), repeat_kv(v, g)
    if scaling is None:
        scaling = q.shape[-1] ** -0.5
    w = torch.matmul(q, ks.transpose(2, 3)) * scaling
    w = torch.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.matmul(w, vs).transpose(1, 2).contiguous()


class CacheLayerOracle:
    """One layer of the reference's cache state machine (packkv_quant.py:45-85): RoPE on K,
    cut whole blocks off the residual, quantise + dequantise them, concatenate."""

    def __init__(self, block: int, recent: int, k_rel: float, v_rel: float, k_mode: str, v_mode: str,
                 high_precision_zero: bool = False):
        self.block, self.recent = block, recent
        self.k_rel, self.v_rel, self.k_mode, self.v_mode = k_rel, v_rel, k_mode, v_mode
        self.hp = high_precision_zero
        self.k_hist = self.v_hist = None
        self.k_res = self.v_res = None

    @staticmethod
    def _cat(a, b):
        if a is None:
            return None if b is None else b.clone()
        return a.clone() if b is None else torch.cat([a, b], dim=2)

    def _step(self, hist, res, new, rel, mode):
        res = self._cat(res, new)
        n = compress_block_count(res.shape[2], self.block, self.recent)
        if n > 0:
            cut = res[:, :, : n * self.block]
            res = res[:, :, n * self.block:]
            c, z, s = quant_ints(cut, self.block, rel, mode, self.hp)
            hist = self._cat(hist, dequant(c, z, s, self.hp))
        return hist, res

    def update(self, k, v, cos, sin):
        k = rope(k, cos, sin)
        self.k_hist, self.k_res = self._step(self.k_hist, self.k_res, k, self.k_rel, self.k_mode)
        self.v_hist, self.v_res = self._step(self.v_hist, self.v_res, v, self.v_rel, self.v_mode)
        return self._cat(self.k_hist, self.k_res), self._cat(self.v_hist, self.v_res)

    def seq_length(self) -> int:
        n = 0 if self.k_hist is None else self.k_hist.shape[2]
        return n + (0 if self.k_res is None else self.k_res.shape[2])
