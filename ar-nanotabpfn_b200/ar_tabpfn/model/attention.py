"""Attention module of the drop-in package.

``MultiheadAttention`` keeps the reference's parameters (four bias-free
projections, ar_tabpfn/model/attention.py:31-43 of the reference) so that
state_dicts load unchanged.  On the inference path these modules are weight
containers: the kernels read their packed weights.  The mask factories return
small descriptions of the visibility (``DenseMask``, ``RowMask``) instead of
flex BlockMasks; ``ARTabPFN.forward`` takes them.
"""
from __future__ import annotations

import torch
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

    @torch.no_grad()
    def forward(self, q, k, v, block_mask):
        """The reference's module call (ar_tabpfn/model/attention.py:45-61) for inference:
        q [B,Sq,D], k / v [B,Skv,D] -> (out [B,Sq,D], (K, V) [B,H,Skv,Dh]).  ``block_mask`` is a
        ``DenseMask`` (every query sees every key: the feature attention across column tokens) or a
        ``RowMask`` (self-attention over rows laid out [context | buffer | other]).  The softmax
        attention runs on this library's kernels; the four projections are plain library GEMMs.
        No autograd graph is built."""
        from . import triton_kernels as tk
        B, Sq, D = q.shape
        Skv = k.shape[1]
        H, Dh = self.n_heads, self.head_dim
        qh = self.q_proj(q).view(B, Sq, H, Dh).transpose(1, 2)
        kh = self.k_proj(k).view(B, Skv, H, Dh).transpose(1, 2)
        vh = self.v_proj(v).view(B, Skv, H, Dh).transpose(1, 2)
        if isinstance(block_mask, RowMask):
            if Sq != Skv or block_mask.num_rows != Sq:
                raise ValueError("a RowMask describes self-attention over num_rows rows")
            out = tk.row_attention(qh, kh, vh, block_mask.context_len, block_mask.buffer_len, block_mask.visible)
        elif isinstance(block_mask, DenseMask):
            out = tk.dense_attention(qh, kh, vh)
        else:
            raise TypeError("block_mask must be a DenseMask or a RowMask of this package (flex BlockMasks are not "
                            "decoded)")
        out = out.transpose(1, 2).reshape(B, Sq, D)
        return self.out_proj(out), (kh, vh)


class DenseMask:
    """What ``create_dense_mask`` / ``create_context_self_attention_mask`` return here: every
    query sees every key, which the kernels do without a mask tensor."""

    def __init__(self, seq_len: int):
        self.seq_len = int(seq_len)


class RowMask:
    """Row-attention visibility of the reference's ``create_row_mask``
    (ar_tabpfn/model/attention.py:86-175) as data instead of a flex BlockMask.

    Every row sees all context rows.  Context rows see nothing else.  The mask over the
    buffer rows is a prefix for every other row, so it is stored as one count per
    non-context row: ``visible[j]`` = how many leading buffer rows row ``context_len + j``
    sees.  Buffer j sees buffers <= j; target t sees buffers <= t mod Nb while
    t < attending_chunks * Nb and no buffer afterwards."""

    def __init__(self, num_rows: int, context_len: int, buffer_len: int, visible):
        self.num_rows, self.context_len, self.buffer_len = int(num_rows), int(context_len), int(buffer_len)
        self.visible = [int(v) for v in visible]
        if len(self.visible) != self.num_rows - self.context_len:
            raise ValueError("one visible count per non-context row is needed")

    @classmethod
    def prefix(cls, context_len: int, buffer_len: int, visible) -> "RowMask":
        """Any mask of the family: ``visible`` lists the counts of the buffer rows, then the target rows."""
        visible = list(visible)
        return cls(context_len + len(visible), context_len, buffer_len, visible)

    @classmethod
    def teacher_forcing(cls, context_len: int, num_targets: int) -> "RowMask":
        """Buffer j sees buffers <= j, target i sees buffers < i (the inference pattern)."""
        return cls.prefix(context_len, num_targets, [j + 1 for j in range(num_targets)] + list(range(num_targets)))


def create_dense_mask(seq_len: int, device=None) -> DenseMask:
    return DenseMask(seq_len)


def create_context_self_attention_mask(context_len: int, device=None) -> DenseMask:
    return DenseMask(context_len)


def create_row_mask(num_rows: int, context_len: int, buffer_len: int, attending_chunks=None,
                    device=None) -> RowMask:
    """Same arguments as the reference factory; returns the visibility as a ``RowMask``."""
    target_len = num_rows - context_len - buffer_len
    if target_len < 0 or buffer_len < 0 or context_len < 0:
        raise ValueError("num_rows must cover the context and buffer rows")
    if attending_chunks is None:
        attending_chunks = target_len // (2 * buffer_len) if buffer_len else 0
    vis = [j + 1 for j in range(buffer_len)]
    for t in range(target_len):
        vis.append((t % buffer_len) + 1 if buffer_len and t < attending_chunks * buffer_len else 0)
    return RowMask(num_rows, context_len, buffer_len, vis)


def clear_mask_cache():
    """No masks are cached: dense and block-causal visibility is computed inside the kernels."""
