"""Shared test plumbing: builds a device CompressedLayer from the CPU oracle's quantiser
output (so kernels under test see exactly the reference's codes, scales and zero-points)."""
import torch

from oracle import quant as Q
from packkv_b200 import ops


def _pad16(n):
    return (n + 15) // 16 * 16


def layer_from_oracle(k, v, *, block, bits_k, bits_v, k_mode, cbk, cbv, rel_k, rel_v, device, hp=False):
    """k, v: CPU (B, Hkv, n_comp, 128) tensors to compress entirely.  Returns
    (CompressedLayer on device, dequantised K, dequantised V on CPU per the reference)."""
    B, H, S, D = k.shape
    kc, kz, ks = Q.quant_ints(k, block, rel_k, k_mode, hp)
    vc, vz, vs = Q.quant_ints(v, block, rel_v, "token", hp)
    kd, vd = Q.dequant(kc, kz, ks, hp), Q.dequant(vc, vz, vs, hp)

    def per_seq_codes(c5):   # (B,H,nb,blk,D) -> (B, S, H*D) u8
        return c5.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous().to(torch.uint8)

    kcodes, vcodes = per_seq_codes(kc).to(device), per_seq_codes(vc).to(device)
    nkb, nvb = (S // cbk) * H, (S // cbv) * 2 * H
    k_stream = torch.zeros(B, _pad16(nkb * ops.block_bound("k", cbk, bits_k)) + 16, dtype=torch.uint8, device=device)
    v_stream = torch.zeros(B, _pad16(nvb * ops.block_bound("v", cbv, bits_v)) + 16, dtype=torch.uint8, device=device)
    k_stream, k_info, k_bytes, f1 = ops.encode_codes("k", kcodes, cbk, bits_k, stream=k_stream)
    v_stream, v_info, v_bytes, f2 = ops.encode_codes("v", vcodes, cbv, bits_v, stream=v_stream)
    assert int(f1.item()) == 0 and int(f2.item()) == 0
    if k_mode == "channel":
        assert block == cbk
        k_scale = ks.reshape(B, H, S // block, D).contiguous().to(device)
        k_zero = kz.reshape(B, H, S // block, D).contiguous().to(device)
    else:
        k_scale = ks.reshape(B, S).contiguous().to(device)
        k_zero = kz.reshape(B, S).contiguous().to(device)
    layer = ops.CompressedLayer(
        k_stream=k_stream, k_info=k_info, k_bytes=k_bytes, k_scale=k_scale, k_zero=k_zero,
        v_stream=v_stream, v_info=v_info, v_bytes=v_bytes,
        v_scale=vs.reshape(B, S).contiguous().to(device), v_zero=vz.reshape(B, S).contiguous().to(device),
        n_comp=S, kv_heads=H, cbk=cbk, cbv=cbv, bits_k=bits_k, bits_v=bits_v,
        k_mode=ops.K_CHANNEL if k_mode == "channel" else ops.K_TOKEN, high_precision_zero=hp)
    return layer, kd, vd
