"""The HuggingFace hook end to end on a GPU: a small random-weight Llama decodes with the
registered custom attention function.  With a masker stack that selects every key
(Sink over the whole sequence -> full mask) the sparse call must reproduce the model's own
eager attention; with a real sparse stack the attention output of layer 0, for the queries, keys
and values the hook was given, must be what the CPU restatement of the reference computes."""

import numpy as np
import pytest
import torch

from sparse_attention_hub.adapters import ModelAdapterHF
from sparse_attention_hub.sparse_attention import (
    HashAttentionTopKMaskerConfig,
    LocalMaskerConfig,
    ResearchAttentionConfig,
    SinkMaskerConfig,
)
import workloads


def _tiny_llama(dtype):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                      max_position_embeddings=512, attn_implementation="eager")
    return LlamaForCausalLM(cfg).to("cuda:0", dtype).eval()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gpu_full_mask_equals_eager_attention(dtype):
    model = _tiny_llama(dtype)
    adapter = ModelAdapterHF("tiny-llama", ResearchAttentionConfig(masker_configs=[SinkMaskerConfig(10 ** 6)]),
                             model=model, tokenizer=None)
    ids = torch.randint(0, 128, (2, 200), device="cuda:0")
    with torch.no_grad():
        ctx = model(ids[:, :192], use_cache=True)
        dense = model(ids[:, 192:], past_key_values=ctx.past_key_values, use_cache=True).logits
        ctx = model(ids[:, :192], use_cache=True)
        with adapter.enable_sparse_mode():
            sparse = model(ids[:, 192:], past_key_values=ctx.past_key_values, use_cache=True,
                           sparse_meta_data={}).logits
    tol = 1e-3 if dtype == torch.float32 else 6e-2
    torch.testing.assert_close(sparse.float(), dense.float(), atol=tol, rtol=tol)


@pytest.mark.gpu
def test_gpu_sparse_stack_decodes_through_the_hook():
    model = _tiny_llama(torch.bfloat16)
    w = workloads.hat_weights(3, 4, 64, 32, 32, 2)
    hat = {layer: {n: [workloads.to_torch(a, "bf16", "cuda:0") for a in arrs] for n, arrs in w.items()}
           for layer in range(2)}
    cfg = ResearchAttentionConfig(masker_configs=[
        SinkMaskerConfig(4), LocalMaskerConfig(16),
        HashAttentionTopKMaskerConfig(heavy_size=0.1, hat_bits=32, hat_mlp_layers=2, hat_mlp_hidden_size=32,
                                      hat_mlp_activation="silu", hat_weights=hat)])
    adapter = ModelAdapterHF("tiny-llama", cfg, model=model, tokenizer=None)
    ids = torch.randint(0, 128, (1, 300), device="cuda:0")
    meta: dict = {}
    # record what the hook hands to layer 0 and what it gets back
    seen = []
    inner = adapter.sparse_attention.custom_attention

    def recording(module, queries, keys, values, attention_mask, scaling, dropout, **kwargs):
        result = inner(module, queries, keys, values, attention_mask, scaling, dropout, **kwargs)
        if kwargs.get("layer_idx") == 0:
            seen.append(tuple(None if t is None else t.detach().float().cpu().numpy()
                              for t in (queries, keys, values, attention_mask, result[0])) + (float(scaling),))
        return result

    adapter.sparse_attention.custom_attention = recording
    with torch.no_grad():
        ctx = model(ids[:, :296], use_cache=True)
        with adapter.enable_sparse_mode():
            out = model(ids[:, 296:], past_key_values=ctx.past_key_values, use_cache=True, sparse_meta_data=meta)
            for _ in range(3):  # decode steps append keys; the signature cache grows with them
                nxt = out.logits[:, -1].argmax(-1, keepdim=True)
                out = model(nxt, past_key_values=out.past_key_values, use_cache=True, sparse_meta_data=meta)
    assert torch.isfinite(out.logits.float()).all()
    assert meta["key"][0].length == 303 and meta["key"][1].length == 303
    # question tokens (Sq = 4, causal mask) and three decode steps, each against the restatement
    from oracle import stacks

    assert [s_[0].shape[2] for s_ in seen] == [4, 1, 1, 1]
    stack = [("sink", {"sink_size": 4}), ("local", {"window_size": 16}),
             ("hash_topk", {"heavy_size": 0.1, "bits": 32, "hidden": 32, "layers": 2, "activation": "silu",
                            "weights": {n: [workloads.to_dtype(a, "bf16") for a in arrs] for n, arrs in w.items()}})]
    for q, k, v, am, got, scaling in seen:
        _, ref_out, _ = stacks.run_stack(stack, q, k, v, scaling, "bf16", attention_mask=am)
        np.testing.assert_allclose(got, ref_out, atol=2e-2, rtol=2e-2)
