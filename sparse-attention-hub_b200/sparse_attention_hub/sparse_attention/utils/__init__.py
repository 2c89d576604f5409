"""Mask container and masked-attention entry points."""

from .mask import Mask

__all__ = ["Mask"]
