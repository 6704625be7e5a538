"""Attention module of the drop-in package.

``MultiheadAttention`` keeps the reference's parameters (four bias-free
projections, ar_tabpfn/model/attention.py:31-43 of the reference) so that
state_dicts load unchanged.  On the inference path these modules are weight
containers: the kernels read their packed weights.  The block-mask factories
of the reference serve its training loop and are not part of this build.
"""
from __future__ import annotations

from torch import nn


class MultiheadAttention(nn.Module):
    def __init__(self, d_model: int, n_heads: int):
        super().__init__()
        self.n_heads = n_heads
        self.head_dim = d_model // n_heads
        self.scale = self.head_dim ** -0.5
        self.q_proj = nn.Linear(d_model, d_model, bias=False)
        self.k_proj = nn.Linear(d_model, d_model, bias=False)
        self.v_proj = nn.Linear(d_model, d_model, bias=False)
        self.out_proj = nn.Linear(d_model, d_model, bias=False)

    def forward(self, *args, **kwargs):
        raise NotImplementedError(
            "the training forward (flex_attention block masks) is outside this build; "
            "use ARTabPFNPredictor for sampling and log-density evaluation")


def _training_only(name):
    def fn(*args, **kwargs):
        raise NotImplementedError(f"{name} builds a training BlockMask and is outside this build")
    fn.__name__ = name
    return fn


create_dense_mask = _training_only("create_dense_mask")
create_row_mask = _training_only("create_row_mask")
create_context_self_attention_mask = _training_only("create_context_self_attention_mask")


def clear_mask_cache():
    """No masks are cached: dense and block-causal visibility is computed inside the kernels."""
