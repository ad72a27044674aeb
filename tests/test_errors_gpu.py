"""GPU: error behaviour of the boundary.  The reference aborts the process on a failed
packkv_assert (include/utils.h:8-16), throws "not supported" for shapes it does not dispatch
(src/k_encode_cpu.cpp:328-330) and silently returns 0.0 from its GPU launchers for unknown shapes
(src/kernels.cu:586-589).  Here every such condition is a status code (-> ValueError /
RuntimeError("not supported")) or a bit in the device flag word; nothing aborts and no kernel
reads or writes outside its buffers."""
import pytest
import torch

from packkv_b200 import _lib, encode, ops, synth
from packkv_b200.config import QuantMode

pytestmark = pytest.mark.gpu


def test_stream_overflow_is_flagged_not_written(cuda_device):
    codes = torch.randint(0, 16, (1, 256, 256), dtype=torch.uint8, device=cuda_device)
    small = torch.full((1, 1024), 0xAB, dtype=torch.uint8, device=cuda_device)      # far too small for 8 blocks
    _, info, nbytes, flags = ops.encode_codes("k", codes, 64, 4, stream=small)
    torch.cuda.synchronize()
    assert int(flags.item()) & _lib.FLAG_STREAM_OVERFLOW
    written = int((small != 0xAB).sum().item())
    assert written <= 1024                                                          # nothing outside the buffer (it has no room to check beyond)


def test_code_out_of_range_is_flagged(cuda_device):
    codes = torch.randint(0, 4, (1, 128, 128), dtype=torch.uint8, device=cuda_device)
    codes[0, 5, 7] = 9                                                              # does not fit 2 bits
    *_, flags = ops.encode_codes("k", codes, 64, 2)
    torch.cuda.synchronize()
    assert int(flags.item()) & _lib.FLAG_CODE_RANGE


def test_constant_channel_is_flagged_by_the_encoder(cuda_device):
    k, v = synth.synth_kv(1, 2, 128, 128, seed=3, dtype=torch.float16, device=cuda_device)
    k[:, :, :, 17] = 0.5                                                            # scale 0: the reference produces NaN codes here
    flags = ops.new_flags(cuda_device)
    encode.compress_kv(k, v, block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14, k_mode=QuantMode.ChannelQuant, flags=flags)
    torch.cuda.synchronize()
    assert int(flags.item()) & _lib.FLAG_CODE_RANGE


def test_corrupt_block_table_is_flagged_by_attention(cuda_device):
    k, v = synth.synth_kv(1, 2, 256, 128, seed=4, dtype=torch.float16, device=cuda_device)
    q = synth.synth_q(1, 8, 128, seed=4, dtype=torch.float16)[:, :, 0].contiguous().to(cuda_device)
    layer = encode.compress_kv(k, v, block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14, k_mode=QuantMode.ChannelQuant)
    good = ops.decode_attention(q, layer, None, None, 0)
    for bad_offset, bad_size in ((1 << 30, None), (None, 1 << 20), (3, None)):     # past the stream, larger than any block, odd
        info = layer.k_info.clone()
        if bad_offset is not None:
            info[0, 1, 0] = bad_offset
        if bad_size is not None:
            info[0, 1, 1] = bad_size
        broken = ops.CompressedLayer(**{**layer.__dict__, "k_info": info})
        flags = ops.new_flags(cuda_device)
        out = ops.decode_attention(q, broken, None, None, 0, flags=flags)
        torch.cuda.synchronize()
        assert int(flags.item()) & _lib.FLAG_BAD_STREAM
        assert out.shape == good.shape
    flags = ops.new_flags(cuda_device)
    again = ops.decode_attention(q, layer, None, None, 0, flags=flags)              # the context is still healthy
    torch.cuda.synchronize()
    assert int(flags.item()) == 0 and torch.equal(again, good)


def test_status_codes_map_to_exceptions(cuda_device):
    codes = torch.zeros(1, 128, 128, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(RuntimeError, match="not supported"):
        ops.encode_codes("k", codes, 64, 5)                                         # bit width the format does not have
    with pytest.raises(RuntimeError, match="not supported"):
        ops.encode_codes("k", codes[:, :96].contiguous(), 48, 4)                                 # token block that is not 32 / 64 / 128
    with pytest.raises(ValueError):
        ops.encode_codes("k", codes[:, :100].contiguous(), 64, 4)                                # context not a multiple of the block
    with pytest.raises(ValueError):
        ops.decode_attention(torch.zeros(1, 8, 96, dtype=torch.float16, device=cuda_device), None, None, None, 0)
    lib = _lib.lib()
    assert lib.pkv_decode_attention(None, None) == _lib.PKV_ERR_BAD_ARGUMENT        # null argument block: a status, not a crash
