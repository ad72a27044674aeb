"""Seeded synthetic K/V/q tensors with the shapes and value distributions of the benchmark
configurations.  They stand in for real-model KV caches, which need checkpoints and prompts
that are not available offline.

K ~ N(0,1) per element, scaled per (head, channel) by lognormal(0, 0.5), with 4 outlier
channels (chosen by a seeded permutation of the head dimension) scaled by 10; optionally
rotated with RoPE (base 10000, positions 0..S-1).  V ~ N(0,1).  q ~ N(0,1).
"""
from __future__ import annotations

import torch


def rope_tables(seq_len: int, head_dim: int, *, base: float = 10000.0, start: int = 0,
                device="cpu", dtype=torch.float32):
    """cos, sin of shape (1, seq_len, head_dim) for positions start..start+seq_len-1."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    pos = torch.arange(start, start + seq_len, dtype=torch.float32, device=device)
    ang = torch.outer(pos, inv)
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(dtype).unsqueeze(0), emb.sin().to(dtype).unsqueeze(0)


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def synth_kv(batch: int, kv_heads: int, seq_len: int, head_dim: int, *, seed: int, dtype=torch.float16,
             device="cpu", apply_rope: bool = False):
    """Returns K, V of shape (batch, kv_heads, seq_len, head_dim) in `dtype` on `device`."""
    g = torch.Generator(device=device).manual_seed(seed)
    k = torch.randn(batch, kv_heads, seq_len, head_dim, generator=g, device=device, dtype=torch.float32)
    chan = torch.exp(0.5 * torch.randn(kv_heads, head_dim, generator=g, device=device, dtype=torch.float32))
    outl = torch.randperm(head_dim, generator=g, device=device)[:4]
    chan[:, outl] *= 10.0
    k = k * chan[None, :, None, :]
    v = torch.randn(batch, kv_heads, seq_len, head_dim, generator=g, device=device, dtype=torch.float32)
    k, v = k.to(dtype), v.to(dtype)
    if apply_rope:
        cos, sin = rope_tables(seq_len, head_dim, device=device, dtype=dtype)
        k = (k * cos.unsqueeze(1)) + (_rotate_half(k) * sin.unsqueeze(1))
    return k, v


def synth_q(batch: int, q_heads: int, head_dim: int, *, seed: int, dtype=torch.float16, device="cpu"):
    """Returns q of shape (batch, q_heads, 1, head_dim)."""
    g = torch.Generator(device=device).manual_seed(seed + 7919)
    return torch.randn(batch, q_heads, 1, head_dim, generator=g, device=device, dtype=torch.float32).to(dtype)


def rel_for_bits(bits: int) -> float:
    """quant_scale_rel that yields codes below 2**bits: the quantiser produces up to
    1/rel + 2 distinct levels, so rel = 1/(2**bits - 2)."""
    return 1.0 / (2 ** bits - 2)
