"""KV-head-sharded decode attention.

On one GPU: the exchange path of the attention launch (rows stored into every rank's gathered buffer, arrival
counters, the bounded wait) with the ranks run one after the other on the same device, and a wait whose
counters never arrive, which must give up with the timeout flag and leave the context usable.
On 2 GPUs (skipped on a single-GPU box): two processes over NCCL, both exchange modes, equal to the single-GPU
result bit for bit."""
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
            # the same through the launch's own peer stores, three steps in a row (the two buffers alternate)
            flags = ops.new_flags(dev)
            x = parallel.HeadExchange(B, (qhi - qlo), world, dtype, dev, mode="peer", rank=rank, kv_heads_local=hi - lo, flags=flags)
            ok = True
            for _ in range(3):
                local = ops.decode_attention(q[:, qlo:qhi].contiguous(), layer, k[:, lo:hi, S:].contiguous(), v[:, lo:hi, S:].contiguous(), R,
                                             flags=flags, exchange=x.begin())
                x.gather(local)
                torch.cuda.synchronize()
                ok = ok and torch.equal(x.full(), want)
                dist.barrier()
            results[(rank, k_mode.value, "peer")] = bool(ok) and int(flags.item()) == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_head_sharded_attention_equals_single_gpu():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == 8 and all(results.values()), dict(results)


@pytest.mark.parametrize("plan", [None, (2, 3, 2)])
def test_exchange_rows_and_counters_on_one_gpu(cuda_device, plan):
    """Two ranks' launches run one after the other on one device, each with the exchange block that names both
    ranks' (local) gathered buffers: the buffers end up equal to the unsharded result and every counter has
    grown by batch * local KV heads; the wait then passes without a poll running out.  Also in the two-launch
    form, where the pair's last cluster to finish delivers the rows."""
    from packkv_b200 import _lib, encode, ops, parallel, synth
    from packkv_b200.config import QuantMode
    dev, dtype = cuda_device, torch.float16
    B, H, G, S, R, world = 2, 4, 2, 256, 20, 2
    k, v = synth.synth_kv(B, H, S + R, 128, seed=5, dtype=dtype, device=dev, apply_rope=True)
    q = synth.synth_q(B, H * G, 128, seed=5, dtype=dtype, device=dev)[:, :, 0].contiguous()
    args = dict(block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14, k_mode=QuantMode.ChannelQuant)
    full = encode.compress_kv(k[:, :, :S], v[:, :, :S], **args)
    scratch = ops.new_attention_scratch(dev) if plan else None
    want = ops.decode_attention(q, full, k[:, :, S:].contiguous(), v[:, :, S:].contiguous(), R, scratch=scratch, plan=plan)
    Hl, Hql = H // world, H * G // world
    gathered = [torch.zeros(world, B, Hql, 128, dtype=dtype, device=dev) for _ in range(world)]
    arrivals = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    flags = ops.new_flags(dev)
    for rank in range(world):
        layer, (lo, hi) = parallel.compress_kv_head_shard(k[:, :, :S], v[:, :, :S], rank, world, **args)
        x = _lib.AttnExchange()
        x.n_ranks, x.rank = world, rank
        for r in range(world):
            x.gathered[r], x.arrivals[r] = gathered[r].data_ptr(), arrivals[r].data_ptr()
        ops.decode_attention(q[:, lo * G:hi * G].contiguous(), layer, k[:, lo:hi, S:].contiguous(), v[:, lo:hi, S:].contiguous(), R,
                             flags=flags, exchange=x, scratch=scratch, plan=plan)
    for r in range(world):
        # (the wait may start while the launch before it drains, so it needs more than a handful of polls)
        ops.exchange_wait(arrivals[r], world, B * Hl, flags, max_polls=1_000_000)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    for r in range(world):
        assert arrivals[r].tolist() == [B * Hl] * world
        assert torch.equal(gathered[r].permute(1, 0, 2, 3).reshape(B, H * G, 128), want)


def test_exchange_wait_gives_up(cuda_device):
    """A rank that never arrives: the wait returns after its poll limit with PKV_FLAG_TIMEOUT set, and the device
    keeps working afterwards."""
    from packkv_b200 import _lib, ops
    dev = cuda_device
    arrivals = torch.zeros(4, dtype=torch.int32, device=dev)
    arrivals[0] = 7
    flags = ops.new_flags(dev)
    ops.exchange_wait(arrivals, 4, 7, flags, max_polls=50)
    torch.cuda.synchronize()
    assert int(flags.item()) == _lib.FLAG_TIMEOUT
    arrivals[:] = 7
    flags.zero_()
    ops.exchange_wait(arrivals, 4, 7, flags, max_polls=50)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0


def test_consuming_wait_serves_every_step(cuda_device):
    """The wait that takes a step's arrivals off the counters again: three steps with the same call, the counters end
    at zero; a step whose arrivals are missing gives up with the flag and takes nothing."""
    from packkv_b200 import _lib, ops
    dev = cuda_device
    arrivals = torch.zeros(4, dtype=torch.int32, device=dev)
    flags = ops.new_flags(dev)
    for _ in range(3):
        arrivals += 6                       # what four ranks' launches would have added
        ops.exchange_wait(arrivals, 4, 6, flags, max_polls=50, consume=True)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0 and arrivals.tolist() == [0, 0, 0, 0]
    arrivals[:3] = 6
    ops.exchange_wait(arrivals, 4, 6, flags, max_polls=50, consume=True)
    torch.cuda.synchronize()
    assert int(flags.item()) == _lib.FLAG_TIMEOUT and arrivals.tolist() == [6, 6, 6, 0]
