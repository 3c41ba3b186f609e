"""B200-native Converse2D / Converse block (drop-in for Yiozolm/ConverseNet's hot path)."""
from .util_converse import Converse2D, ConverseBlock, ConverseBlockAlphaVariant, LayerNorm, sequential  # noqa: F401
from . import _cabi  # noqa: F401

__all__ = ["Converse2D", "ConverseBlock", "ConverseBlockAlphaVariant", "LayerNorm", "sequential"]
