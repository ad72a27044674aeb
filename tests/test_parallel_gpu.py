"""GPU, 2 ranks over NCCL (skipped on a single-GPU box): KV-head-sharded decode attention with an
all-gather of the outputs equals the single-GPU result bit for bit, and every rank's streams are the
per-head slices of the single-GPU encoding."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from packkv_b200 import encode, ops, parallel, synth
        from packkv_b200.config import QuantMode
        B, H, G, S, R = 2, 4, 4, 512, 130
        dtype = torch.bfloat16
        k, v = synth.synth_kv(B, H, S + R, 128, seed=3, dtype=dtype, device=dev, apply_rope=True)
        q = synth.synth_q(B, H * G, 128, seed=3, dtype=dtype, device=dev)[:, :, 0].contiguous()
        args = dict(block=128, bits_k=2, bits_v=4, k_rel=synth.rel_for_bits(2), v_rel=synth.rel_for_bits(4))
        for k_mode in (QuantMode.ChannelQuant, QuantMode.TokenQuant):
            full = encode.compress_kv(k[:, :, :S], v[:, :, :S], k_mode=k_mode, **args)
            want = ops.decode_attention(q, full, k[:, :, S:].contiguous(), v[:, :, S:].contiguous(), R)
            layer, (lo, hi) = parallel.compress_kv_head_shard(k[:, :, :S], v[:, :, :S], rank, world, k_mode=k_mode, **args)
            qlo, qhi = parallel.q_heads_of(lo, hi, G)
            local = ops.decode_attention(q[:, qlo:qhi].contiguous(), layer, k[:, lo:hi, S:].contiguous(), v[:, lo:hi, S:].contiguous(), R)
            got = parallel.gather_heads(local)
            torch.cuda.synchronize()
            ok = torch.equal(got, want)
            results[(rank, k_mode.value)] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_head_sharded_attention_equals_single_gpu():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == 4 and all(results.values()), dict(results)
