"""Host-side plumbing of `jointqk_b200.hf` under a real `transformers` model on the CPU: the cache
layer protocol (prefill, one-token steps, lengths, mask sizes), the registered attention function
and `generate()`.  The paged cache is replaced by a dense stand-in that attends exactly, so the
logits must equal those of the stock path up to the bf16 rounding of the query; the kernels themselves are covered by the GPU tests."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


class DensePaged:
    """What the cache layer needs of PagedKVCache, kept dense and exact."""

    def __init__(self, tables, n_seqs, v_tables=None):
        self.k = self.v = None
        self.steps = 0

    def prefill(self, k, v):
        self.k, self.v = k.float(), v.float()

    def generate_step(self, k_new, v_new, q, own_key_exact=False):
        self.steps += 1
        self.k = torch.cat([self.k, k_new.float()], 2)
        self.v = torch.cat([self.v, v_new.float()], 2)
        g = q.shape[1] // self.k.shape[1]
        kk, vv = self.k.repeat_interleave(g, 1), self.v.repeat_interleave(g, 1)
        s = torch.einsum("bhd,bhtd->bht", q.float(), kk) / q.shape[-1] ** 0.5
        return torch.einsum("bht,bhtd->bhd", s.softmax(-1), vv)


def _tiny(family: str):
    """The two model families the reference evaluates (Llama-3.1 and Qwen3 attention), at toy size."""
    import transformers as tf

    kw = dict(vocab_size=128, hidden_size=256, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, max_position_embeddings=256)
    if family == "llama":
        return tf.LlamaForCausalLM(tf.LlamaConfig(**kw)).eval()
    return tf.Qwen3ForCausalLM(tf.Qwen3Config(**kw)).eval()


@torch.no_grad()
@pytest.mark.parametrize("family", ["llama", "qwen3"])
def test_cache_layer_and_attention_function_under_generate(monkeypatch, family):
    from transformers import cache_utils

    from jointqk_b200 import hf

    monkeypatch.setattr(hf, "PagedKVCache", DensePaged)
    torch.manual_seed(0)
    model = _tiny(family)
    ids = torch.randint(0, 128, (2, 24))
    kw = dict(max_new_tokens=6, do_sample=False, output_logits=True, return_dict_in_generate=True, pad_token_id=0,
              attention_mask=torch.ones_like(ids))
    ref = model.generate(ids, **kw)

    hf.set_attention(model)
    assert model.config._attn_implementation == hf.ATTN_NAME
    layer_cls = hf.make_paged_layer_class()
    layers = []
    for m in hf.attention_modules(model):
        if m.layer_idx == 0:                                   # layer 0 at full precision: the stock dense layer
            layers.append(cache_utils.DynamicLayer())
            m._jqk_layer = None
        else:
            layers.append(layer_cls(None))
            m._jqk_layer = layers[-1]
    cache = cache_utils.Cache(layers=layers)
    got = model.generate(ids, past_key_values=cache, **kw)

    assert torch.equal(ref.sequences, got.sequences)
    scale = max(a.abs().max().item() for a in ref.logits)
    assert max((a - b).abs().max().item() for a, b in zip(ref.logits, got.logits)) < 5e-3 * scale   # the step takes q in bf16
    for layer in layers[1:]:
        assert layer.get_seq_length() == 24 + 5 and layer.paged.steps == 5      # the last token is never fed back
        assert layer.get_mask_sizes(1) == (30, 0)
        assert layer.take_pending() is None
    with pytest.raises(NotImplementedError):
        layers[1].update(torch.zeros(2, 2, 3, 64), torch.zeros(2, 2, 3, 64))    # chunked prefill
    with pytest.raises(NotImplementedError):
        layers[1].reorder_cache(torch.tensor([0, 1]))
    layers[1].reset()
    assert layers[1].get_seq_length() == 0 and layers[1].get_mask_sizes(7) == (7, 0)
