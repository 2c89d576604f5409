"""Request / response types and the adapter interfaces (reference: adapters/base.py:11-115)."""

from abc import ABC, abstractmethod
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generator, List, Union

from ..sparse_attention.base import SparseAttention, SparseAttentionConfig


@dataclass
class Request:
    """A context that is prefilled once with dense attention, and one or more questions
    answered on top of it with sparse attention."""

    context: str
    questions: Union[str, List[str]]
    answer_prefix: str = ""


@dataclass
class RequestResponse:
    """One response per question (a bare string when a bare question was asked)."""

    responses: Union[str, List[str]]


class ModelHubAdapterInterface(ABC):
    @abstractmethod
    def process_request(self, request: Request, generation_kwargs: Dict[str, Any],
                        request_kwargs: Dict[str, Any]) -> RequestResponse:
        ...


class SparseAttentionAdapterInterface(ABC):
    @abstractmethod
    def get_custom_attention_function(self, sparse_attention: SparseAttention) -> Callable:
        ...


class ModelAdapter(SparseAttentionAdapterInterface, ModelHubAdapterInterface, ABC):
    """Holds the sparse-attention object built from its config (None config = dense only)."""

    def __init__(self, model_name: str, sparse_attention_config, **kwargs: Any) -> None:
        self.model_name = model_name
        self.sparse_attention_config = sparse_attention_config
        self.sparse_attention = (SparseAttention.create_from_config(sparse_attention_config)
                                 if sparse_attention_config is not None else None)

    @abstractmethod
    @contextmanager
    def enable_sparse_mode(self) -> Generator[None, None, None]:
        ...
