"""Model components (same public names as the reference's ar_tabpfn.model)."""

from .model import ARTabPFN, Embedder, TwoStageTransformer, TwoStageTransformerLayer, MixtureGaussianHead
from .attention import (MultiheadAttention, create_dense_mask, create_row_mask,
                        create_context_self_attention_mask, clear_mask_cache)
from .triton_kernels import triton_available, cross_attention
from .inference import ARTabPFNPredictor

__all__ = [
    "ARTabPFN", "Embedder", "TwoStageTransformer", "TwoStageTransformerLayer", "MixtureGaussianHead",
    "ARTabPFNPredictor", "MultiheadAttention", "create_dense_mask", "create_row_mask",
    "create_context_self_attention_mask", "clear_mask_cache", "triton_available", "cross_attention",
]
