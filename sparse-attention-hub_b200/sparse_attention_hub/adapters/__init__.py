"""Adapters between this package and model hosting libraries."""

from .base import (
    ModelAdapter,
    ModelHubAdapterInterface,
    Request,
    RequestResponse,
    SparseAttentionAdapterInterface,
)
from .huggingface import ModelAdapterHF

__all__ = ["Request", "RequestResponse", "ModelHubAdapterInterface", "SparseAttentionAdapterInterface",
           "ModelAdapter", "ModelAdapterHF"]
