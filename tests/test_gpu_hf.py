"""The packed cache under a real `transformers` model: a small random-weight Llama decodes through
`jointqk_b200.hf` (calibrate -> fit -> packed cache layers -> one fused launch per layer and step)
and its logits are compared, step by step on the same forced tokens, with the same model run the
reference's way: a dense cache whose keys are replaced by the oracle's reconstruction after the
layer's forward (prefill keys after prefill, a decode key after the step that produced it; Mode B
of experiments/stage1/toolkit/jointqk_press.py:275-308), stock attention over it."""

import pytest
import torch

pytestmark = pytest.mark.gpu

transformers = pytest.importorskip("transformers")

from oracle import reference_port as orc  # noqa: E402


def _model(family="llama"):
    """Random weights, the attention shapes of the two families the reference evaluates."""
    import transformers as tf

    torch.manual_seed(1234)
    kw = dict(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, max_position_embeddings=1024)
    model = tf.LlamaForCausalLM(tf.LlamaConfig(**kw)) if family == "llama" else tf.Qwen3ForCausalLM(tf.Qwen3Config(**kw))
    return model.to(device="cuda", dtype=torch.bfloat16).eval()


def _oracle_layer_class(comps):
    """Dense cache layer with the reference's Mode-B bookkeeping, keys through the oracle."""
    from transformers.cache_utils import DynamicLayer

    class OracleLayer(DynamicLayer):
        def update(self, key_states, value_states, *args, **kwargs):
            if not self.is_initialized:
                self.lazy_initialization(key_states, value_states)
            keys = torch.cat([self.keys, key_states], dim=-2)          # what this step's attention sees: new keys exact
            self.values = torch.cat([self.values, value_states], dim=-2)
            recon = torch.stack([
                torch.stack([orc.roundtrip(key_states[b, h].float().cpu(), comps[h].codebooks_padded, comps[h].forward_map,
                                           comps[h].inverse_map)[0] for h in range(key_states.shape[1])])
                for b in range(key_states.shape[0])]).to(key_states)
            self.keys = torch.cat([self.keys, recon], dim=-2)           # what later steps see
            return keys, self.values

    return OracleLayer


@torch.no_grad()
@pytest.mark.parametrize("family", ["llama", "qwen3"])
def test_model_decodes_over_the_packed_cache_like_the_reference_flow(family):
    from transformers import cache_utils

    from jointqk_b200 import hf, paged

    model = _model(family)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 512, (2, 256), generator=g).cuda() for _ in range(4)]
    moments = hf.calibrate(model, prompts)
    assert float(moments.tokens.min()) == 4 * 2 * 256
    cache = hf.build_cache(model, moments, k_bits=2.0)
    assert isinstance(cache.layers[0], cache_utils.DynamicLayer) and len(cache.layers) == 3

    ids = torch.randint(0, 512, (2, 48), generator=g).cuda()
    forced = torch.randint(0, 512, (2, 12), generator=g).cuda()

    def run(past):
        out = [model(input_ids=ids, past_key_values=past, use_cache=True).logits[:, -1].float()]
        for t in range(forced.shape[1]):
            out.append(model(input_ids=forced[:, t:t + 1], past_key_values=past, use_cache=True).logits[:, -1].float())
        return torch.stack(out)

    hf.OWN_KEY_EXACT = True
    got = run(cache)
    for L in (1, 2):
        layer = cache.layers[L]
        assert layer.paged.lengths == [48 + 12] * 2 and layer.get_seq_length() == 60
        paged.check_status(layer.paged.status)

    # the same model the reference's way
    for m in hf.attention_modules(model):
        m._jqk_layer = None
    oracle_layers = [cache_utils.DynamicLayer()] + [_oracle_layer_class(cache.jqk_compressors[L])() for L in (1, 2)]
    want = run(cache_utils.Cache(layers=oracle_layers))

    # and without any compression, to show that the comparison is not vacuous
    plain = run(cache_utils.DynamicCache())

    scale = want.abs().max().item()
    err = (got - want).abs().max().item() / scale
    effect = (plain - want).abs().max().item() / scale
    mean_err = (got - want).abs().mean().item() / scale
    mean_effect = (plain - want).abs().mean().item() / scale
    print(f"logits: packed vs reference flow {err:.3e} (mean {mean_err:.3e}), compression effect {effect:.3e} (mean {mean_effect:.3e})")
    assert torch.allclose(got[0], want[0], atol=1e-5 * scale)        # prefill sees exact keys in both
    assert err < 2e-2                                               # bf16 logits resolve 4e-3; 16-bit tables, bf16 weights in P.V
    assert mean_effect > 2 * mean_err                                # the comparison is not vacuous (means: a bf16 ulp is coarse for maxima)


@torch.no_grad()
@pytest.mark.parametrize("cap", [4, 8])
def test_llama_decodes_with_keys_and_values_packed(cap):
    """K at 2 bits and V at 3 bits, the reference's usual pairing: values calibrated through the
    model's forward (first and second moments), packed by the centred eigenbasis compressor, and the
    decode step attends over both code pools.  Checked against the same model over a dense cache
    whose keys and values are the oracle's reconstructions, the new token's included (with packed
    values the step compresses the new row before it attends)."""
    from transformers import cache_utils
    from transformers.cache_utils import DynamicLayer

    from jointqk_b200 import hf, paged

    model = _model()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 512, (2, 256), generator=g).cuda() for _ in range(4)]
    moments = hf.calibrate(model, prompts, with_values=True)
    cache = hf.build_cache(model, moments, k_bits=2.0, v_bits=3, max_bits=cap)   # 8: the reference's own cap
    ids = torch.randint(0, 512, (2, 40), generator=g).cuda()
    forced = torch.randint(0, 512, (2, 6), generator=g).cuda()

    def run(past):
        out = [model(input_ids=ids, past_key_values=past, use_cache=True).logits[:, -1].float()]
        for t in range(forced.shape[1]):
            out.append(model(input_ids=forced[:, t:t + 1], past_key_values=past, use_cache=True).logits[:, -1].float())
        return torch.stack(out)

    got = run(cache)
    for L in (1, 2):
        assert cache.layers[L].paged.v_tables is not None and cache.layers[L].paged.lengths == [46, 46]
        paged.check_status(cache.layers[L].paged.status)

    def oracle_layer(kc, vc):
        class OracleLayer(DynamicLayer):
            def update(self, key_states, value_states, *args, **kwargs):
                if not self.is_initialized:
                    self.lazy_initialization(key_states, value_states)
                rk = torch.stack([torch.stack([orc.roundtrip(key_states[b, h].float().cpu(), kc[h].codebooks_padded, kc[h].forward_map,
                                                             kc[h].inverse_map)[0] for h in range(key_states.shape[1])])
                                  for b in range(key_states.shape[0])]).to(key_states)
                rv = torch.stack([torch.stack([orc.centred_roundtrip(value_states[b, h].float().cpu(), vc[h].mu, vc[h].inner.codebooks_padded,
                                                                     vc[h].inner.forward_map, vc[h].inner.inverse_map)[0]
                                               for h in range(value_states.shape[1])])
                                  for b in range(value_states.shape[0])]).to(value_states)
                first = self.keys.numel() == 0
                self.keys = torch.cat([self.keys, rk], dim=-2)
                self.values = torch.cat([self.values, rv], dim=-2)
                # prefill attends over the exact rows (the pages are filled behind it), a step over the stored ones
                return (key_states, value_states) if first else (self.keys, self.values)
        return OracleLayer()

    for m in hf.attention_modules(model):
        m._jqk_layer = None
    want = run(cache_utils.Cache(layers=[DynamicLayer()] + [oracle_layer(cache.jqk_compressors[L], cache.jqk_v_compressors[L])
                                                             for L in (1, 2)]))
    plain = run(cache_utils.DynamicCache())
    scale = want.abs().max().item()
    err = (got - want).abs().max().item() / scale
    effect = (plain - want).abs().max().item() / scale
    print(f"logits, K 2 bits + V 3 bits: packed vs reference flow {err:.3e}, compression effect {effect:.3e}")
    assert err < 2e-2 and effect > 2 * err
