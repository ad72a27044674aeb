"""The cache and the fused decode attention inside an unmodified transformers model.

A randomly initialised Llama-shaped model (no checkpoint) is run twice over the same tokens:
once with dense dequantised K/V and the library's eager attention at every step -- what the
reference's patched models do (models/llama.py:259-282) -- and once with decode steps served by
the fused decompress-attention kernel through the registered attention function.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("family", ["mistral", "qwen3", "phi3"])
def test_other_model_families(family):
    """The same drop-in on the other families the reference patches (models/mistral.py, qwen3.py, phi.py); Phi-3
    has head_dim 96 and no grouped queries, its cache is created with hidden_size // num_attention_heads
    (models/phi.py:744-747)."""
    transformers = pytest.importorskip("transformers")
    from packkv_b200 import hf
    from packkv_b200.cache import PackKVCacheConfigStatic
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, RepackMethod
    kw = dict(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, intermediate_size=1024,
              vocab_size=1000, head_dim=128, max_position_embeddings=1024)
    if family == "mistral":
        from transformers import MistralConfig as Cfg, MistralForCausalLM as Model
        kw["sliding_window"] = None
    elif family == "phi3":
        from transformers import Phi3Config as Cfg, Phi3ForCausalLM as Model
        kw = dict(hidden_size=384, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=2, intermediate_size=768,
                  vocab_size=1000, max_position_embeddings=1024, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    else:
        from transformers import Qwen3Config as Cfg, Qwen3ForCausalLM as Model
    torch.manual_seed(2)
    cfg = Cfg(**kw)
    model = Model(cfg).to("cuda", torch.bfloat16).eval()
    hf.register()
    model.set_attn_implementation(hf.ATTN_NAME)
    PackKVCacheConfigStatic.config = PackKVCacheConfig(family, QuantMethod.KIVI, RepackMethod.MEDIAN, False, 64, 192, 16, 1 / 14, 1 / 14)
    ids = torch.randint(0, 1000, (2, 300), device="cuda")

    def run(materialize):
        cache = hf.make_cache(cfg, 2, materialize=materialize)
        outs = []
        with torch.no_grad():
            outs.append(model(ids[:, :280], past_key_values=cache, use_cache=True).logits[:, -1:])
            for t in range(280, 300):
                outs.append(model(ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits)
        cache.check_flags()
        return torch.cat(outs, 1).float()

    ref, got = run(True), run(False)
    assert ((got - ref).abs().max() / ref.abs().max()).item() < 2e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_llama_decode_through_registered_attention(dtype):
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from packkv_b200 import hf
    from packkv_b200.cache import PackKVCacheConfigStatic
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, RepackMethod

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2,
                      intermediate_size=1024, vocab_size=2000, head_dim=128, max_position_embeddings=1024)
    model = LlamaForCausalLM(cfg).to("cuda", dtype).eval()
    hf.register()
    model.set_attn_implementation(hf.ATTN_NAME)
    PackKVCacheConfigStatic.config = PackKVCacheConfig("llama", QuantMethod.KIVI, RepackMethod.NONE, False, 64, 192, 16, 1 / 14, 1 / 14)
    B, prefill, steps = 3, 330, 70
    ids = torch.randint(0, 2000, (B, prefill + steps), device="cuda")

    def run(materialize):
        cache = hf.make_cache(cfg, B, materialize=materialize)
        outs = []
        with torch.no_grad():
            outs.append(model(ids[:, :prefill], past_key_values=cache, use_cache=True).logits[:, -1:])
            for t in range(prefill, prefill + steps):
                outs.append(model(ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits)
        assert cache.get_seq_length() == prefill + steps
        cache.check_flags()
        return torch.cat(outs, 1).float(), cache

    ref, _ = run(True)
    got, cache = run(False)
    assert cache._layers[0].n_comp >= 192          # the decode steps crossed block boundaries
    err = (got - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, float(err)
    # greedy decoding picks the same tokens wherever the reference's margin is not a near tie
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 4 * (got - ref).abs().max()
    assert bool((got.argmax(-1) == ref.argmax(-1))[clear].all())


def test_generate_runs():
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from packkv_b200 import hf
    from packkv_b200.cache import PackKVCacheConfigStatic
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, RepackMethod

    torch.manual_seed(1)
    cfg = LlamaConfig(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=2,
                      intermediate_size=512, vocab_size=500, head_dim=128, max_position_embeddings=1024)
    model = LlamaForCausalLM(cfg).to("cuda", torch.float16).eval()
    hf.register()
    model.set_attn_implementation(hf.ATTN_NAME)
    PackKVCacheConfigStatic.config = PackKVCacheConfig("llama", QuantMethod.KIVI, RepackMethod.NONE, False, 64, 192, 16, 1 / 14, 1 / 14)
    ids = torch.randint(3, 500, (2, 260), device="cuda")
    cache = hf.make_cache(cfg, 2)
    out = model.generate(ids, attention_mask=torch.ones_like(ids), past_key_values=cache, max_new_tokens=6, do_sample=False)
    assert out.shape == (2, 266)
    assert cache.get_seq_length() == 265          # the last generated token is not fed back


@pytest.mark.parametrize("family", ["llama", "phi3"])
def test_every_decode_attention_against_oracle_on_the_dense_view(family):
    """Inside a running transformers model: every fused decode attention call (both layers, steps that cross a
    block boundary included) is compared at 2e-3 with the reference's eager attention (oracle, CPU) over the
    cache's dense view, which the cache tests pin to the reference cache bit for bit."""
    transformers = pytest.importorskip("transformers")
    from oracle import quant as Q
    from packkv_b200 import hf
    from packkv_b200.cache import PackKVCacheConfigStatic
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, RepackMethod
    dtype = torch.bfloat16
    torch.manual_seed(3)
    if family == "llama":
        from transformers import LlamaConfig as Cfg, LlamaForCausalLM as Model
        cfg = Cfg(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, intermediate_size=1024, vocab_size=2000,
                  head_dim=128, max_position_embeddings=1024)
    else:
        from transformers import Phi3Config as Cfg, Phi3ForCausalLM as Model
        cfg = Cfg(hidden_size=384, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=2, intermediate_size=768, vocab_size=1000,
                  max_position_embeddings=1024, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    model = Model(cfg).to("cuda", dtype).eval()
    hf.register()
    model.set_attn_implementation(hf.ATTN_NAME)
    PackKVCacheConfigStatic.config = PackKVCacheConfig(family, QuantMethod.KIVI, RepackMethod.NONE, False, 64, 192, 16, 1 / 14, 1 / 14)
    B, prefill, steps = 2, 300, 40
    ids = torch.randint(3, 1000, (B, prefill + steps), device="cuda")
    cache = hf.make_cache(cfg, B)
    inner, worst, calls = cache.attend, [0.0], [0]

    def checked(query_states, layer_idx, scaling=None):
        out = inner(query_states, layer_idx, scaling)                       # (B, 1, Hq, D)
        kd, vd = cache.dense(layer_idx)
        ref = Q.eager_attention(query_states.cpu(), kd.cpu(), vd.cpu(), scaling)   # (B, 1, Hq, D)
        err = ((out.float().cpu() - ref.float()).abs().max() / ref.float().abs().max()).item()
        worst[0], calls[0] = max(worst[0], err), calls[0] + 1
        return out
    cache.attend = checked
    try:
        with torch.no_grad():
            model(ids[:, :prefill], past_key_values=cache, use_cache=True)
            for t in range(prefill, prefill + steps):
                model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
        cache.check_flags()
    finally:
        PackKVCacheConfigStatic.config = None
    assert calls[0] == 2 * steps
    assert worst[0] <= 2e-3, worst[0]
