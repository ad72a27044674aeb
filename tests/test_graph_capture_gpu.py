"""GPU: the decode entry points inside a CUDA graph.  They allocate nothing, never synchronise and launch on
the stream they are given, so a decode step (every layer's fused attention, single launch or the two-launch
form with its scratch, the append folded in) can be captured once and replayed with new inputs written in
place, which is how a serving loop removes the per-launch host cost."""
import pytest
import torch

from packkv_b200 import encode, ops, synth
from packkv_b200.config import QuantMode

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("plan", [None, (4, 2, 2)])
def test_decode_step_replays_from_a_graph(cuda_device, plan):
    dev, dtype = cuda_device, torch.bfloat16
    B, Hkv, G, n_comp, n_res, layers = 2, 2, 4, 1024, 140, 3
    built = []
    for li in range(layers):
        k, v = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=60 + li, dtype=dtype, device=dev, apply_rope=True)
        layer = encode.compress_kv(k[:, :, :n_comp], v[:, :, :n_comp], block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14,
                                   k_mode=QuantMode.ChannelQuant, cbk=64, cbv=128)
        k_res = torch.zeros(B, Hkv, 256, 128, dtype=dtype, device=dev)
        v_res = torch.zeros_like(k_res)
        k_res[:, :, :n_res - 1], v_res[:, :, :n_res - 1] = k[:, :, n_comp:-1], v[:, :, n_comp:-1]
        built.append((layer, k_res, v_res, k[:, :, -1:].contiguous(), v[:, :, -1:].contiguous()))
    cos, sin = synth.rope_tables(1, 128, start=n_comp + n_res - 1, device=dev, dtype=dtype)
    q = [synth.synth_q(B, Hkv * G, 128, seed=70 + li, dtype=dtype, device=dev)[:, :, 0].contiguous() for li in range(layers)]
    out = [torch.empty_like(x) for x in q]
    flags = ops.new_flags(dev)
    scratch = ops.new_attention_scratch(dev) if plan else None

    def step():
        for (layer, k_res, v_res, k_new, v_new), qi, oi in zip(built, q, out):
            ops.decode_attention(qi, layer, k_res, v_res, n_res, out=oi, flags=flags, append=(k_new, v_new, cos, sin), scratch=scratch, plan=plan)

    step()                                    # eager: also the first-use set-up of the library (function attributes)
    torch.cuda.synchronize()
    want_first = [o.clone() for o in out]
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.current_stream().wait_stream(side)
    for o in out:
        o.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    for o, w in zip(out, want_first):
        assert torch.equal(o, w)
    # new queries written in place: the replay must equal the eager launch on the same data
    for qi in q:
        qi.copy_(torch.roll(qi, 1, dims=1) * 0.5)
    graph.replay()
    torch.cuda.synchronize()
    got = [o.clone() for o in out]
    step()
    torch.cuda.synchronize()
    for g_, o in zip(got, out):
        assert torch.equal(g_, o)
    assert int(flags.item()) == 0
