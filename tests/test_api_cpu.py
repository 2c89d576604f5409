"""Host-side behaviour of the reference API that needs no GPU: config validation, the masker
registry, error types, Mask semantics on CPU tensors, and the rule that the native path has
no CPU fallback."""

import pytest
import torch

from sparse_attention_hub import _native
from sparse_attention_hub.adapters import ModelAdapterHF, Request, RequestResponse
from sparse_attention_hub.sparse_attention import (
    AdaptiveSamplingMaskerConfig,
    HashAttentionTopKMaskerConfig,
    LocalMaskerConfig,
    MagicPigConfig,
    Mask,
    OracleTopKConfig,
    PQCacheConfig,
    RandomSamplingMaskerConfig,
    ResearchAttention,
    ResearchAttentionConfig,
    SinkMaskerConfig,
    SparseAttention,
)
from sparse_attention_hub.sparse_attention.research_attention.maskers.base import MaskerRegistry


def test_config_validation_matches_the_reference():
    with pytest.raises(ValueError):
        LocalMaskerConfig(window_size=0)
    with pytest.raises(ValueError):
        SinkMaskerConfig(sink_size=-1)
    with pytest.raises(ValueError):
        RandomSamplingMaskerConfig(sampling_rate=0.0)
    with pytest.raises(ValueError):
        AdaptiveSamplingMaskerConfig(base_rate_sampling=1.5, epsilon=0.1, delta=0.1, init_offset=0, local_offset=0)
    with pytest.raises(ValueError):
        AdaptiveSamplingMaskerConfig(base_rate_sampling=0.1, epsilon=1.0, delta=0.1, init_offset=0, local_offset=0)
    with pytest.raises(ValueError):
        MagicPigConfig(lsh_l=0, lsh_k=4)
    with pytest.raises(ValueError):
        MagicPigConfig(lsh_l=4, lsh_k=65)
    with pytest.raises(ValueError):
        MagicPigConfig(lsh_l=4, lsh_k=4, packing="int8")


def test_registry_routes_configs_to_maskers():
    ra = ResearchAttention.create_from_config(ResearchAttentionConfig(masker_configs=[
        SinkMaskerConfig(4), LocalMaskerConfig(8), OracleTopKConfig(heavy_size=0.1),
        MagicPigConfig(lsh_l=4, lsh_k=4)]))
    assert [type(m).__name__ for m in ra.maskers] == ["SinkMasker", "LocalMasker", "OracleTopK", "MagicPig"]
    assert isinstance(SparseAttention.create_from_config(ResearchAttentionConfig(masker_configs=[])),
                      ResearchAttention)
    assert PQCacheConfig in MaskerRegistry.get_all_registered_types()
    assert HashAttentionTopKMaskerConfig in MaskerRegistry.get_all_registered_types()


def test_error_types():
    with pytest.raises(ValueError):  # at most one sampling masker
        ResearchAttention.create_from_config(ResearchAttentionConfig(masker_configs=[
            RandomSamplingMaskerConfig(0.1), MagicPigConfig(lsh_l=4, lsh_k=4)]))
    ra = ResearchAttention.create_from_config(ResearchAttentionConfig(masker_configs=[SinkMaskerConfig(4)]))
    q = torch.zeros(1, 2, 1, 8)
    k = torch.zeros(1, 2, 16, 8)
    with pytest.raises(ValueError):  # sparse_meta_data is mandatory
        ra.custom_attention(None, q, k, k, None, 1.0, 0.0)
    with pytest.raises(TypeError):
        ResearchAttention.create_from_config(SinkMaskerConfig(4))


def test_native_path_has_no_cpu_fallback():
    ra = ResearchAttention.create_from_config(ResearchAttentionConfig(masker_configs=[SinkMaskerConfig(4)]))
    q = torch.zeros(1, 2, 1, 8)
    k = torch.zeros(1, 2, 16, 8)
    with pytest.raises(_native.NativeLibraryError):
        ra.custom_attention(None, q, k, k, None, 1.0, 0.0, sparse_meta_data={}, layer_idx=0)


def test_mask_semantics_on_cpu_tensors():
    shape = (1, 1, 2, 6)
    dense = torch.tensor([[[[0.0, 0.5, 0.0, 1.0, 0.0, 0.0], [0.25, 0.0, 0.0, 0.0, 0.0, 1.0]]]])
    m = Mask.create_mask_from_dense_mask(shape, dense, dtype=torch.float32)
    idx, ptr, data = m.get_index_mask()
    assert idx.tolist() == [1, 3, 6, 11] and ptr.tolist() == [0, 2, 4]  # flat row * n + col
    assert data.tolist() == [0.5, 1.0, 0.25, 1.0]
    again = Mask.create_mask_from_indices(shape, idx, ptr, data, dtype=torch.float32)
    assert torch.equal(again.get_dense_mask(), dense)
    merged = m.merge_mask(Mask.create_mask_from_dense_mask(shape, dense, torch.float32), inplace=False)
    assert torch.equal(merged.get_dense_mask(), torch.clamp(dense * 2, 0, 1))
    x = torch.ones(shape)
    inv = m.apply_inv_mask(x)
    assert torch.allclose(inv[0, 0, 0, 1], torch.tensor(1.0 / (0.5 + 1e-6))) and inv[0, 0, 0, 0] == 0
    assert Mask.create_full_mask(shape, torch.float32, "cpu").is_full_mask()
    empty = Mask.create_empty_mask(shape, torch.float32, "cpu")
    assert empty.is_empty_mask() and torch.equal(empty.apply_inv_mask(x), x)
    assert empty.merge_mask(m, inplace=False).get_density() == pytest.approx(4 / 12)
    rw = Mask.create_from_row_wise_idx(shape, torch.tensor([[[[1, 1], [5, 0]]]]), torch.full((1, 1, 2, 2), 0.5),
                                       mask_type="index", dtype=torch.float32, mode="sparse")
    assert rw.get_index_mask()[1].tolist() == [0, 2, 4]  # duplicates kept in the sparse form
    rw = Mask.create_from_row_wise_idx(shape, torch.tensor([[[[1, 1], [5, 0]]]]), torch.full((1, 1, 2, 2), 0.5),
                                       mask_type="dense", dtype=torch.float32)
    assert rw.get_index_mask()[1].tolist() == [0, 1, 3]  # and collapsed by the dense scatter


class _RecordingAttention(ResearchAttention):
    def __init__(self):
        super().__init__(sparse_attention_config=ResearchAttentionConfig(masker_configs=[]), maskers=[])
        self.calls = []

    def custom_attention(self, module, queries, keys, values, attention_mask, scaling, dropout, **kwargs):
        self.calls.append(kwargs)
        return queries.transpose(1, 2), None


def test_hf_hook_closure_and_sparse_mode():
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    model = LlamaForCausalLM(cfg)
    adapter = ModelAdapterHF("tiny-llama", ResearchAttentionConfig(masker_configs=[SinkMaskerConfig(4)]),
                             model=model, tokenizer=None)
    rec = _RecordingAttention()
    hook = adapter.get_custom_attention_function(rec)
    layer = model.model.layers[1].self_attn
    q = torch.zeros(1, 4, 1, 8)
    with pytest.raises(ValueError):
        hook(layer, q, q, q, None)
    out, w = hook(layer, q, q, q, None, scaling=0.5, sparse_meta_data={"a": 1})
    assert out.shape == (1, 1, 4, 8) and w is None
    assert rec.calls[0]["layer_idx"] == 1 and rec.calls[0]["sparse_meta_data"] == {"a": 1}

    before = model.config._attn_implementation
    with adapter.enable_sparse_mode():
        name = model.config._attn_implementation
        assert name.startswith("sparse_attention_") and name in ALL_ATTENTION_FUNCTIONS.valid_keys()
    assert model.config._attn_implementation == before
    adapter._cleanup_attention_registration()
    assert name not in ALL_ATTENTION_FUNCTIONS.valid_keys()
    dense_only = ModelAdapterHF("tiny-llama", None, model=model, tokenizer=None)
    with pytest.raises(RuntimeError):
        with dense_only.enable_sparse_mode():
            pass
    assert Request("c", "q").answer_prefix == "" and RequestResponse("r").responses == "r"
