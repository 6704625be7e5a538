"""B200-native drop-in for the AR-TabPFN sampling / log-density path.

Import names follow the reference package (``ar_tabpfn.model.ARTabPFN``,
``ar_tabpfn.model.ARTabPFNPredictor`` ...).  The data generators and the
training loop of the reference are not part of this build.
"""

from .model import (ARTabPFN, Embedder, TwoStageTransformer, TwoStageTransformerLayer, MixtureGaussianHead,
                    MultiheadAttention, ARTabPFNPredictor, create_dense_mask, create_row_mask,
                    create_context_self_attention_mask, clear_mask_cache, triton_available, cross_attention)

__all__ = [
    "ARTabPFN", "Embedder", "TwoStageTransformer", "TwoStageTransformerLayer", "MixtureGaussianHead",
    "MultiheadAttention", "ARTabPFNPredictor", "create_dense_mask", "create_row_mask",
    "create_context_self_attention_mask", "clear_mask_cache", "triton_available", "cross_attention",
]
