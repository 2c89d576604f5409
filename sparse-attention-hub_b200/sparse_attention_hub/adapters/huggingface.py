"""HuggingFace transformers adapter: the custom-attention hook and sparse mode.

Reference: adapters/huggingface.py (hook closure :227-275, registration :277-343,
enable_sparse_mode :345-386, request processing :120-225, generation :388-490).

transformers calls an attention implementation looked up by name in
`ALL_ATTENTION_FUNCTIONS` as
`fn(module, queries, keys, values, attention_mask, scaling=..., dropout=..., **kwargs)` and
reshapes its first result as `[B, Sq, Hq * D]`.  The hook registered here forwards that
call to `SparseAttention.custom_attention`, adding the module's `layer_idx`, and insists on
the caller-owned `sparse_meta_data` dict that the maskers keep their per-layer state in.
The additive-mask builder registered under the same name is transformers' `eager_mask`.
Loading of weights goes through transformers directly (`from_pretrained`) unless a model
object is handed in; there is no process-wide model server here.
"""

import random
import string
from contextlib import contextmanager
from typing import Any, Callable, Dict, Generator, List, Optional, Tuple

import torch

from ..sparse_attention.base import SparseAttention
from ..sparse_attention.research_attention.base import ResearchAttention
from .base import ModelAdapter, Request, RequestResponse


def _registries():
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    return ALL_ATTENTION_FUNCTIONS, ALL_MASK_ATTENTION_FUNCTIONS


class ModelAdapterHF(ModelAdapter):
    """Runs a causal LM with dense prefill of the context and sparse decoding of questions."""

    def __init__(self, model_name: str, sparse_attention_config, model_kwargs: Optional[Dict[str, Any]] = None,
                 tokenizer_kwargs: Optional[Dict[str, Any]] = None, device: Optional[str] = None,
                 model: Optional[torch.nn.Module] = None, tokenizer: Any = None, **kwargs: Any) -> None:
        super().__init__(model_name, sparse_attention_config, **kwargs)
        self._registered_attention_name: Optional[str] = None
        self._custom_attention_fn: Optional[Callable] = None
        self._sparse_attention_available = sparse_attention_config is not None
        self.device = device
        if model is None:
            from transformers import AutoModelForCausalLM, AutoTokenizer

            model = AutoModelForCausalLM.from_pretrained(model_name, **(model_kwargs or {}))
            if device is not None:
                model = model.to(device)
            if tokenizer is None:
                tokenizer = AutoTokenizer.from_pretrained(model_name, **(tokenizer_kwargs or {}))
                if tokenizer.pad_token is None:
                    tokenizer.pad_token = tokenizer.eos_token
        self.model = model
        self.tokenizer = tokenizer

    def __del__(self) -> None:
        try:
            self._cleanup_attention_registration()
        except Exception:
            pass

    # ------------------------------------------------------------------ the hook
    def get_custom_attention_function(self, sparse_attention: SparseAttention) -> Callable:
        def custom_attention_callable(module: torch.nn.Module, queries: torch.Tensor, keys: torch.Tensor,
                                      values: torch.Tensor, attention_mask: Optional[torch.Tensor],
                                      scaling: float = 1.0, dropout: float = 0.0,
                                      **kwargs: Dict[str, Any]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
            layer_idx = getattr(module, "layer_idx", None)
            if layer_idx is not None:
                kwargs["layer_idx"] = layer_idx
            if "sparse_meta_data" not in kwargs:
                raise ValueError("sparse_meta_data must be provided while calling model.forward()")
            sparse_meta_data = kwargs.pop("sparse_meta_data")
            return sparse_attention.custom_attention(
                module=module, queries=queries, keys=keys, values=values, attention_mask=attention_mask,
                scaling=scaling, dropout=dropout, sparse_meta_data=sparse_meta_data, **kwargs)

        return custom_attention_callable

    def _generate_unique_attention_name(self) -> str:
        attn, masks = _registries()
        taken = set(attn.valid_keys()) | set(masks.valid_keys())
        while True:
            name = "sparse_attention_" + "".join(random.choices(string.ascii_lowercase + string.digits, k=8))
            if name not in taken:
                return name

    def _ensure_attention_registered(self) -> str:
        if self._registered_attention_name is None:
            if not self._sparse_attention_available or self.sparse_attention is None:
                raise RuntimeError("Cannot register attention function: sparse attention is not available")
            if not isinstance(self.sparse_attention, ResearchAttention):
                raise NotImplementedError("Sparse attention is not supported for this model yet")
            from transformers.masking_utils import eager_mask

            attn, masks = _registries()
            self._custom_attention_fn = self.get_custom_attention_function(self.sparse_attention)
            self._registered_attention_name = self._generate_unique_attention_name()
            attn.register(self._registered_attention_name, self._custom_attention_fn)
            masks.register(self._registered_attention_name, eager_mask)
        return self._registered_attention_name

    def _cleanup_attention_registration(self) -> None:
        name = self._registered_attention_name
        if name is not None:
            for registry in _registries():
                if name in registry.valid_keys():
                    registry._global_mapping.pop(name, None)
        self._registered_attention_name = None
        self._custom_attention_fn = None

    @contextmanager
    def enable_sparse_mode(self) -> Generator[None, None, None]:
        """Every module whose config carries `_attn_implementation` runs the hook inside the block."""
        if not self._sparse_attention_available:
            raise RuntimeError("Cannot enable sparse mode: sparse attention is not available")
        original: Dict[str, str] = {}
        for name, module in self.model.named_modules():
            if hasattr(module, "config") and hasattr(module.config, "_attn_implementation"):
                original[name] = module.config._attn_implementation
        hook_name = self._ensure_attention_registered()
        try:
            for name, module in self.model.named_modules():
                if name in original:
                    module.config._attn_implementation = hook_name
            yield
        finally:
            for name, module in self.model.named_modules():
                if name in original:
                    module.config._attn_implementation = original[name]

    # ------------------------------------------------------------------ requests
    def process_request(self, request: Request, generation_kwargs: Dict[str, Any],
                        request_kwargs: Dict[str, Any], **kwargs: Any) -> RequestResponse:
        """Dense prefill of the context, then each question decoded greedily in sparse mode on a
        copy-free rewind of the context cache (adapters/huggingface.py:120-225)."""
        if self.tokenizer is None:
            raise ValueError("Tokenizer not initialized")
        max_context_length = request_kwargs.get("max_context_length", 2 ** 31 - 1)
        questions: List[str] = [request.questions] if isinstance(request.questions, str) else list(request.questions)
        dev = next(self.model.parameters()).device
        ctx = self.tokenizer.encode(request.context, return_tensors="pt").to(dev)[:, :max_context_length]
        with torch.no_grad():
            context_outputs = self.model(ctx, past_key_values=None, use_cache=True)
        n_ctx = ctx.shape[1]
        responses: List[str] = []
        for question in questions:
            sparse_meta_data: Dict[Any, Any] = {}
            q_tokens = self.tokenizer.encode(question + request.answer_prefix, return_tensors="pt",
                                             add_special_tokens=False).to(dev)
            if self._sparse_attention_available:
                with self.enable_sparse_mode():
                    text = self._generate_response(q_tokens, context_outputs, sparse_meta_data,
                                                   generation_kwargs, **kwargs)
            else:
                text = self._generate_response(q_tokens, context_outputs, sparse_meta_data,
                                               generation_kwargs, **kwargs)
            responses.append(text)
            cache = context_outputs.past_key_values
            if hasattr(cache, "crop"):
                cache.crop(n_ctx)  # drop the question's and the answer's keys again
        return RequestResponse(responses=responses[0] if isinstance(request.questions, str) else responses)

    def _generate_response(self, question_tokens: torch.Tensor, context_outputs: Any,
                           sparse_meta_data: Dict[Any, Any], generation_kwargs: Dict[str, Any],
                           **kwargs: Any) -> str:
        max_new_tokens = int(generation_kwargs.get("max_new_tokens", 50))
        stop_ids = self.model.generation_config.eos_token_id
        stop_ids = stop_ids if isinstance(stop_ids, list) else [stop_ids]
        extra = {"sparse_meta_data": sparse_meta_data} if self._sparse_attention_available else {}
        cache = context_outputs.past_key_values
        with torch.no_grad():
            out = self.model(input_ids=question_tokens, past_key_values=cache, use_cache=True, **extra)
        generated = [out.logits[0, -1].argmax()]
        for _ in range(max_new_tokens - 1):
            if generated[-1].item() in stop_ids:
                break
            with torch.no_grad():
                out = self.model(input_ids=generated[-1].reshape(1, 1), past_key_values=out.past_key_values,
                                 use_cache=True, **extra)
            generated.append(out.logits[0, -1].argmax())
        return self.tokenizer.decode(torch.stack(generated), skip_special_tokens=True)
