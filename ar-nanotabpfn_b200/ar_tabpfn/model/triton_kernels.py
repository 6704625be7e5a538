"""Functional shared-context attention operators, same names and tensor shapes as
the reference module ``ar_tabpfn/model/triton_kernels.py`` (347-475, 478-524,
662-767), executed by the sm_100a kernels of libartab_b200.so.

Shapes follow the reference: q [B,H,Lq,Dh], k_ctx / v_ctx [H,Nc,Dh] shared by the
whole batch, k_buf / v_buf [B,H,Nb,Dh] private per batch element.  Inputs may be
non-contiguous views.  float32 inputs use fp32 FMA kernels, bfloat16 inputs the
tcgen05 tensor-core kernel (head_dim 32) with fp32 accumulation.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _lib


last_status = None


def triton_available() -> bool:
    """True when the CUDA library can be used (the name is the reference's)."""
    try:
        _lib.lib()
        return True
    except Exception:
        return False


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def _rows(q: Tensor) -> Tensor:
    """[B,H,Lq,Dh] -> token-major [B*Lq,H,Dh], contiguous."""
    B, H, Lq, Dh = q.shape
    return q.permute(0, 2, 1, 3).reshape(B * Lq, H, Dh).contiguous()


def _unrows(o: Tensor, B: int, Lq: int) -> Tensor:
    rows, H, Dh = o.shape
    return o.view(B, Lq, H, Dh).permute(0, 2, 1, 3)


def pack_context(k_ctx: Tensor, v_ctx: Tensor) -> Tuple[Tensor, Tensor, int, int]:
    """Lay [H,Nc,Dh] (or [G,H,Nc,Dh]) context K/V out as the kernels read it:
    K [G,H,Ncp,Dh]; V the same in fp32; in bf16 transposed with a hi and a lo part,
    [G,H,2*Dh,Ncp] (the lo part is zero for values that are already bf16)."""
    if k_ctx.dim() == 3:
        k_ctx, v_ctx = k_ctx.unsqueeze(0), v_ctx.unsqueeze(0)
    G, H, Nc, Dh = k_ctx.shape
    Ncp = _pad8(Nc)
    k = torch.zeros(G, H, Ncp, Dh, device=k_ctx.device, dtype=k_ctx.dtype)
    k[:, :, :Nc] = k_ctx
    if k_ctx.dtype == torch.bfloat16:
        v = torch.zeros(G, H, 2 * Dh, Ncp, device=k_ctx.device, dtype=k_ctx.dtype)
        v[:, :, :Dh, :Nc] = v_ctx.transpose(-1, -2)
    else:
        v = torch.zeros(G, H, Ncp, Dh, device=k_ctx.device, dtype=k_ctx.dtype)
        v[:, :, :Nc] = v_ctx
    return k, v, Nc, Ncp


def _context_partials(qr: Tensor, k: Tensor, v: Tensor, Nc: int, Ncp: int, rows_per_group: int,
                      n_splits: int) -> Tuple[Tensor, Tensor]:
    lib = _lib.lib()
    rows, H, Dh = qr.shape
    G = k.shape[0]
    out = torch.empty(n_splits, rows, H, Dh, device=qr.device, dtype=torch.float32)
    lse = torch.empty(n_splits, rows, H, device=qr.device, dtype=torch.float32)
    global last_status
    status = torch.zeros(1, device=qr.device, dtype=torch.int32)
    last_status = status  # non-zero after the launch completes = a bounded device-side wait gave up
    _lib.check(lib.artab_context_attention(_lib.dtype_code(qr.dtype), _lib.ptr(qr), _lib.ptr(k), _lib.ptr(v), rows,
                                           rows_per_group, G, H, Dh, Nc, Ncp, n_splits, _lib.ptr(out),
                                           _lib.ptr(lse), _lib.ptr(status), _lib.stream_ptr()))
    return out, lse


def dense_attention(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """Softmax attention of every query over all keys of its own group: q [G,H,Lq,Dh],
    k / v [G,H,Lk,Dh] -> [G,H,Lq,Dh] (q dtype).  What the reference's MultiheadAttention computes
    under create_dense_mask (ar_tabpfn/model/attention.py:45-61, 72-83), e.g. the feature attention
    across the C column tokens of a row."""
    G, H, Lq, Dh = q.shape
    kp, vp, Nk, Nkp = pack_context(k.to(q.dtype), v.to(q.dtype))
    o, _ = _context_partials(_rows(q), kp, vp, Nk, Nkp, Lq, 1)
    return _unrows(o[0], G, Lq).to(q.dtype)


def row_attention(q: Tensor, k: Tensor, v: Tensor, context_len: int, buffer_len: int, visible) -> Tensor:
    """Self-attention over R rows laid out [context | buffer | other] under a row mask of the
    create_row_mask family (ar_tabpfn/model/attention.py:86-175): q / k / v [G,H,R,Dh] -> [G,H,R,Dh].
    Context rows see the context.  Non-context row j sees the context and the first ``visible[j]``
    buffer rows: its context part and its buffer part are computed separately and merged by
    log-sum-exp in registers (no mask tensor, no concatenated K/V)."""
    G, H, R, Dh = q.shape
    Nc, Nb = int(context_len), int(buffer_len)
    Nr = R - Nc
    if Nc <= 0:
        raise ValueError("row attention needs at least one context row")
    if len(visible) != Nr:
        raise ValueError("one visible count per non-context row is needed")
    lib = _lib.lib()
    kp, vp, _, Ncp = pack_context(k[:, :, :Nc].to(q.dtype), v[:, :, :Nc].to(q.dtype))
    out = torch.empty(G, H, R, Dh, device=q.device, dtype=q.dtype)
    o, _ = _context_partials(_rows(q[:, :, :Nc]), kp, vp, Nc, Ncp, Nc, 1)
    out[:, :, :Nc] = _unrows(o[0], G, Nc).to(q.dtype)
    if Nr > 0:
        qr = _rows(q[:, :, Nc:])
        o, l = _context_partials(qr, kp, vp, Nc, Ncp, Nr, 1)
        kv = _pack_buffer(k[:, :, Nc:Nc + Nb].to(q.dtype), v[:, :, Nc:Nc + Nb].to(q.dtype)) if Nb else None
        vis = torch.tensor([int(x) for x in visible], dtype=torch.int32, device=q.device)
        merged = torch.empty(G * Nr, H, Dh, device=q.device, dtype=torch.float32)
        _lib.check(lib.artab_buffer_attention_merge_visible(
            _lib.dtype_code(q.dtype), _lib.ptr(qr), _lib.ptr(kv), G, H, Dh, Nb, Nr, _lib.ptr(vis), Nb, None,
            _lib.ptr(o), _lib.ptr(l), 1, G * Nr, _lib.ptr(merged), None, _lib.stream_ptr()))
        out[:, :, Nc:] = _unrows(merged, G, Nr).to(q.dtype)
    return out


def _scaled(q: Tensor, scale: Optional[float]) -> Tensor:
    Dh = q.shape[-1]
    if scale is None or abs(scale - Dh ** -0.5) < 1e-12:
        return q
    return q * (scale * Dh ** 0.5)


def triton_context_attention(q: Tensor, k_ctx: Tensor, v_ctx: Tensor,
                             scale: Optional[float] = None, n_splits: int = 1) -> Tuple[Tensor, Tensor]:
    """out [B,H,Lq,Dh] (q dtype), lse [B,H,Lq] fp32 (natural log)."""
    B, H, Lq, Dh = q.shape
    k, v, Nc, Ncp = pack_context(k_ctx.to(q.dtype), v_ctx.to(q.dtype))
    qr = _rows(_scaled(q, scale))
    o, l = _context_partials(qr, k, v, Nc, Ncp, B * Lq, n_splits)
    if n_splits > 1:
        zeros = torch.zeros_like(qr)
        merged = torch.empty(B * Lq, H, Dh, device=q.device, dtype=torch.float32)
        _lib.check(_lib.lib().artab_buffer_attention_merge(
            _lib.dtype_code(q.dtype), _lib.ptr(zeros), None, B * Lq, H, Dh, 0, 0, 1, 0, _lib.ptr(o), _lib.ptr(l),
            n_splits, B * Lq, _lib.ptr(merged), _lib.stream_ptr()))
        lse = torch.logsumexp(l, dim=0)
        return _unrows(merged, B, Lq).to(q.dtype), lse.view(B, Lq, H).permute(0, 2, 1)
    return _unrows(o[0], B, Lq).to(q.dtype), l[0].view(B, Lq, H).permute(0, 2, 1)


def triton_context_attention_multiq(q, k_ctx, v_ctx, scale=None):
    return triton_context_attention(q, k_ctx, v_ctx, scale=scale)


def merge_attention_outputs(out_ctx: Tensor, lse_ctx: Tensor, out_buf: Tensor, lse_buf: Tensor) -> Tensor:
    """Log-sum-exp merge of two partial attentions, [B,H,Lq,Dh] / [B,H,Lq]."""
    B, H, Lq, Dh = out_ctx.shape
    o = torch.stack([_rows(out_ctx.float()), _rows(out_buf.float())])
    l = torch.stack([lse_ctx.float().permute(0, 2, 1).reshape(B * Lq, H),
                     lse_buf.float().permute(0, 2, 1).reshape(B * Lq, H)]).contiguous()
    zeros = torch.zeros(B * Lq, H, Dh, device=out_ctx.device, dtype=torch.float32)
    merged = torch.empty_like(zeros)
    _lib.check(_lib.lib().artab_buffer_attention_merge(
        _lib.F32, _lib.ptr(zeros), None, B * Lq, H, Dh, 0, 0, 1, 0, _lib.ptr(o), _lib.ptr(l), 2, B * Lq,
        _lib.ptr(merged), _lib.stream_ptr()))
    return _unrows(merged, B, Lq).to(out_ctx.dtype)


def _pack_buffer(k_buf: Tensor, v_buf: Tensor) -> Tensor:
    """[B,H,Nb,Dh] x2 -> [B,H,Nb,2,Dh] (K row and V row of a key adjacent)."""
    return torch.stack([k_buf, v_buf], dim=3).contiguous()


def _stream_lengths(mask: Optional[Tensor], B: int, H: int, Lq: int, Nb: int, device) -> Optional[Tensor]:
    """A buffer mask (True = visible, broadcastable to [B,H,Lq,Nb]) as per-stream lengths [B] int32
    when it is one visible prefix per stream (ragged buffers: what the reference itself uses on this
    path, and the fast tensor-core form of the buffer pass); None for any other pattern, which
    ``_buffer_merge_masked`` serves."""
    m = mask.to(device=device, dtype=torch.bool).expand(B, H, Lq, Nb)
    lens = m[:, 0, 0].sum(dim=-1)
    want = torch.arange(Nb, device=device)[None, None, None, :] < lens[:, None, None, None]
    if not torch.equal(m, want.expand(B, H, Lq, Nb)):
        return None
    return lens.to(torch.int32).contiguous()


def _buffer_merge_masked(q: Tensor, kv: Tensor, mask: Tensor, partials, want_lse: bool):
    """The general form: any boolean mask broadcastable to [B,H,Lq,Nb].  One work item per
    (stream, head, query); the mask travels as one byte per (query row, head, key)."""
    lib = _lib.lib()
    B, H, Lq, Dh = q.shape
    Nb = kv.shape[2]
    qr = _rows(q)                                                   # [B*Lq, H, Dh]
    o, l, splits = partials(qr, Lq)
    m = mask.to(device=q.device, dtype=torch.bool).expand(B, H, Lq, Nb)
    km = m.permute(0, 2, 1, 3).reshape(B * Lq, H, Nb).to(torch.uint8).contiguous()
    vis = torch.full((Lq,), Nb, dtype=torch.int32, device=q.device)
    merged = torch.empty(B * Lq, H, Dh, device=q.device, dtype=torch.float32)
    lse = torch.empty(B * Lq, H, device=q.device, dtype=torch.float32) if want_lse else None
    _lib.check(lib.artab_buffer_attention_merge_visible(
        _lib.dtype_code(q.dtype), _lib.ptr(qr), _lib.ptr(kv), B, H, Dh, Nb, Lq, _lib.ptr(vis), Nb, _lib.ptr(km),
        _lib.ptr(o), _lib.ptr(l), splits, B * Lq, _lib.ptr(merged), _lib.ptr(lse), _lib.stream_ptr()))
    return _unrows(merged, B, Lq), (lse.view(B, Lq, H).permute(0, 2, 1) if want_lse else None)


def _buffer_merge(q: Tensor, kv: Tensor, lens: Optional[Tensor], partials, want_lse: bool):
    """Buffer pass + LSE merge for queries q [B,H,Lq,Dh] over packed private K/V [B,H,Nb,2,Dh];
    ``partials(qr, n)`` returns the context partials (o, l, n_splits) of n queries per stream."""
    lib = _lib.lib()
    B, H, Lq, Dh = q.shape
    Nb = kv.shape[2]
    outs, lses = [], []
    for j0 in range(0, Lq, 2):
        n = min(2, Lq - j0)
        qr = _rows(q[:, :, j0:j0 + n])
        o, l, splits = partials(qr, n)
        merged = torch.empty(B * n, H, Dh, device=q.device, dtype=torch.float32)
        lse = torch.empty(B * n, H, device=q.device, dtype=torch.float32) if want_lse else None
        _lib.check(lib.artab_buffer_attention_merge_ragged(
            _lib.dtype_code(q.dtype), _lib.ptr(qr), _lib.ptr(kv) if Nb else None, B, H, Dh, Nb, n, _lib.ptr(lens),
            Nb, _lib.ptr(o), _lib.ptr(l), splits, B * n, _lib.ptr(merged), _lib.ptr(lse), _lib.stream_ptr()))
        outs.append(_unrows(merged, B, n))
        if want_lse:
            lses.append(lse.view(B, n, H).permute(0, 2, 1))
    return torch.cat(outs, dim=2), (torch.cat(lses, dim=2) if want_lse else None)


def pytorch_buffer_attention(q: Tensor, k_buf: Tensor, v_buf: Tensor, mask: Optional[Tensor] = None,
                             scale: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """Attention of q [B,H,Lq,Dh] over each stream's private K/V [B,H,Nb,Dh] -> out (q dtype),
    lse [B,H,Lq] fp32.  ``mask``: any boolean tensor broadcastable to [B,H,Lq,Nb] (True = visible);
    one visible prefix per stream (ragged buffers) takes the fast form of the pass.  A query that
    sees nothing gets out = 0 and lse = -inf, like the reference (triton_kernels.py:570-614).
    The name is the reference's; the work runs in the buffer-pass kernel."""
    B, H, Lq, Dh = q.shape
    Nb = k_buf.shape[2]
    lens = _stream_lengths(mask, B, H, Lq, Nb, q.device) if mask is not None else None
    kv = _pack_buffer(k_buf.to(q.dtype), v_buf.to(q.dtype))

    def no_context(qr, n):
        return (torch.zeros(1, B * n, H, Dh, device=q.device, dtype=torch.float32),
                torch.full((1, B * n, H), float("-inf"), device=q.device, dtype=torch.float32), 1)

    if mask is not None and lens is None and Nb > 0:
        out, lse = _buffer_merge_masked(_scaled(q, scale), kv, mask, no_context, want_lse=True)
    else:
        out, lse = _buffer_merge(_scaled(q, scale), kv, lens, no_context, want_lse=True)
    return out.to(q.dtype), lse


def pytorch_context_attention(q: Tensor, k_ctx: Tensor, v_ctx: Tensor,
                              scale: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """The reference's eager form of the context attention (triton_kernels.py:532-567); here the
    same kernel as ``triton_context_attention``."""
    return triton_context_attention(q, k_ctx, v_ctx, scale=scale)


def hybrid_attention(q: Tensor, k_ctx: Tensor, v_ctx: Tensor, k_buf: Tensor, v_buf: Tensor,
                     buf_mask: Optional[Tensor] = None, use_triton: bool = True) -> Tensor:
    """Shared-context attention + private-buffer attention merged by log-sum-exp.  Every query
    sees every buffer key of its stream, or with ``buf_mask`` (any boolean tensor broadcastable to
    [B,H,Lq,Nb]) what the mask lets it see.  Returns [B,H,Lq,Dh]."""
    B, H, Lq, Dh = q.shape
    Nb = k_buf.shape[2]
    if Nb == 0:
        return triton_context_attention(q, k_ctx, v_ctx)[0]
    lib = _lib.lib()
    lens = _stream_lengths(buf_mask, B, H, Lq, Nb, q.device) if buf_mask is not None else None
    k, v, Nc, Ncp = pack_context(k_ctx.to(q.dtype), v_ctx.to(q.dtype))
    kv = _pack_buffer(k_buf.to(q.dtype), v_buf.to(q.dtype))

    def context(qr, n):
        splits = lib.artab_plan_splits(_lib.dtype_code(q.dtype), B * n, n, 1, H, Nc)
        o, l = _context_partials(qr, k, v, Nc, Ncp, n, splits)
        return o, l, splits

    if buf_mask is not None and lens is None:
        return _buffer_merge_masked(q, kv, buf_mask, context, want_lse=False)[0].to(q.dtype)
    return _buffer_merge(q, kv, lens, context, want_lse=False)[0].to(q.dtype)


def hybrid_teacher_forcing_attention(q: Tensor, k_ctx: Tensor, v_ctx: Tensor, k_buf: Tensor, v_buf: Tensor,
                                     num_targets: int, use_triton: bool = True) -> Tensor:
    """q [B,H,2Nt,Dh] ordered [buffers, targets]; buffer i sees buffer keys <= i,
    target i sees buffer keys < i; everyone sees the whole shared context."""
    B, H, L2, Dh = q.shape
    if L2 != 2 * num_targets:
        raise ValueError("Expected 2*num_targets queries for teacher forcing.")
    if k_buf.shape[2] != num_targets:
        raise ValueError("Expected buffer length to match num_targets.")
    lib = _lib.lib()
    k, v, Nc, Ncp = pack_context(k_ctx.to(q.dtype), v_ctx.to(q.dtype))
    kv = _pack_buffer(k_buf.to(q.dtype), v_buf.to(q.dtype))
    qr = _rows(q)
    splits = lib.artab_plan_splits(_lib.dtype_code(q.dtype), B * L2, L2, 1, H, Nc)
    o, l = _context_partials(qr, k, v, Nc, Ncp, L2, splits)
    merged = torch.empty(B * L2, H, Dh, device=q.device, dtype=torch.float32)
    _lib.check(lib.artab_buffer_attention_merge(
        _lib.dtype_code(q.dtype), _lib.ptr(qr), _lib.ptr(kv), B, H, Dh, num_targets, 1, num_targets, 0,
        _lib.ptr(o), _lib.ptr(l), splits, B * L2, _lib.ptr(merged), _lib.stream_ptr()))
    return _unrows(merged, B, L2).to(q.dtype)


def cross_attention(q: Tensor, k_ctx: Tensor, v_ctx: Tensor, use_triton: bool = True) -> Tensor:
    """Shared-context attention without the LSE output."""
    return triton_context_attention(q, k_ctx, v_ctx)[0]
