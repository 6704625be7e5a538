"""CPU oracle for the AR-TabPFN sampling / log-density hot path.

TEST INFRASTRUCTURE ONLY.  This file is a CPU restatement (torch CPU tensor
ops, no CUDA) of the reference algorithm and exists to check the CUDA path.
Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it; the shipped package never does.

Parity pin: every function below is checked against outputs of the real
reference implementation (golden vectors under ``tests/golden`` produced by
``tests/golden/make_golden.py`` importing the reference package) in
``tests/test_oracle_golden.py``.

Reference locations restated here (paths inside the reference project):
  * ar_tabpfn/model/model.py:51-76        Embedder.embed_{context,buffer,target}
  * ar_tabpfn/model/model.py:190-272      MixtureGaussianHead parameterise / sample / log-likelihood
  * ar_tabpfn/model/triton_kernels.py:478-524   merge_attention_outputs
  * ar_tabpfn/model/triton_kernels.py:532-567   pytorch_context_attention
  * ar_tabpfn/model/triton_kernels.py:570-614   pytorch_buffer_attention
  * ar_tabpfn/model/triton_kernels.py:620-637   teacher-forcing buffer mask
  * ar_tabpfn/model/triton_kernels.py:662-755   hybrid (teacher forcing) attention
  * ar_tabpfn/model/inference.py:181-223, 633-685   shared-context prefill
  * ar_tabpfn/model/inference.py:226-320, 746-833   decode step
  * ar_tabpfn/model/inference.py:323-366            sample_sequence
  * ar_tabpfn/model/inference.py:392-420, 835-890   teacher-forced joint density
  * ar_tabpfn/model/inference.py:423-453, 500-577   per-batch ("flex") semantics
  * ar_tabpfn/model/model.py:317-369, ar_tabpfn/model/attention.py:86-175
                                          training forward under create_row_mask (inference only)

The model is addressed through its ``state_dict`` (a plain ``dict`` of CPU
tensors with the reference's parameter names) so the oracle needs neither the
reference package nor the shipped package.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

MARKER_TARGET, MARKER_CONTEXT, MARKER_BUFFER = 0, 1, 2  # model.py:36-38
LN_EPS = 1e-5
STD_MIN = 1e-3  # model.py:164
STD_MAX = 2.0   # model.py:200


# --------------------------------------------------------------------------
# small pieces
# --------------------------------------------------------------------------

def _bf16_round(x: Tensor) -> Tensor:
    """Round to the nearest bf16-representable value, keep dtype."""
    return x.to(torch.bfloat16).to(x.dtype)


def layer_norm(x: Tensor, w: Tensor, b: Tensor) -> Tensor:
    """nn.LayerNorm over the last axis, eps 1e-5 (model.py:96-98, 138)."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + LN_EPS) * w + b


def gelu_erf(x: Tensor) -> Tensor:
    """nn.GELU() default: exact erf form (model.py:93, 174)."""
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None) -> Tensor:
    y = x @ w.t()
    return y if b is None else y + b


def embed_rows(sd: Dict[str, Tensor], x: Tensor, y: Optional[Tensor], marker: int,
               ar_index: Optional[Tensor] = None) -> Tensor:
    """Embedder.embed_* (model.py:51-76) in closed form.

    x: [..., F]; y: [...] or None; returns [..., D].
    Linear(1, D) applied per feature then averaged over the features equals
    ``mean_F(x) * w_x + b_x``; the oracle keeps the reference's order (apply,
    then average) so that rounding matches.
    """
    wx = sd["embedder.x_embed.weight"][:, 0]
    bx = sd["embedder.x_embed.bias"]
    emb = (x.unsqueeze(-1) * wx + bx).mean(dim=-2)
    if y is not None:
        wy = sd["embedder.y_embed.weight"][:, 0]
        by = sd["embedder.y_embed.bias"]
        emb = emb + (y.unsqueeze(-1) * wy + by)
    emb = emb + sd["embedder.marker_embed.weight"][marker]
    if ar_index is not None:
        emb = emb + sd["ar_tokens"][ar_index]
    return emb


# --------------------------------------------------------------------------
# attention operators (functional; tensors in, tensors out)
# --------------------------------------------------------------------------

def context_attention(q: Tensor, k_ctx: Tensor, v_ctx: Tensor,
                      scale: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """Queries of every stream against one shared context K/V.

    q [B,H,Lq,Dh]; k_ctx, v_ctx [H,Nc,Dh] -> out [B,H,Lq,Dh], lse [B,H,Lq] fp32
    (triton_kernels.py:532-567).
    """
    if scale is None:
        scale = q.shape[-1] ** -0.5
    scores = torch.matmul(q, k_ctx.unsqueeze(0).transpose(-2, -1)) * scale
    lse = torch.logsumexp(scores.float(), dim=-1)
    out = torch.matmul(torch.softmax(scores, dim=-1), v_ctx.unsqueeze(0))
    return out, lse


def buffer_attention(q: Tensor, k_buf: Tensor, v_buf: Tensor,
                     mask: Optional[Tensor] = None,
                     scale: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """Per-stream attention over the private buffer K/V.

    q [B,H,Lq,Dh]; k_buf, v_buf [B,H,Nb,Dh]; mask broadcastable to
    [B,H,Lq,Nb] (True = visible).  Rows with no visible key give out = 0 and
    lse = -inf (triton_kernels.py:570-614).
    """
    if scale is None:
        scale = q.shape[-1] ** -0.5
    scores = torch.matmul(q, k_buf.transpose(-2, -1)) * scale
    dead = None
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
        dead = ~mask.any(dim=-1)
    lse = torch.logsumexp(scores.float(), dim=-1)
    p = torch.softmax(scores, dim=-1)
    if dead is not None:
        p = torch.where(dead.unsqueeze(-1), torch.zeros_like(p), p)
    return torch.matmul(p, v_buf), lse


def teacher_forcing_buffer_mask(num_targets: int) -> Tensor:
    """[1,1,2Nt,Nt] visibility of buffer keys (triton_kernels.py:620-637).

    Query rows 0..Nt-1 are buffer tokens (see keys <= own index), rows
    Nt..2Nt-1 are target tokens (see keys < own index)."""
    qi = torch.arange(2 * num_targets)
    kj = torch.arange(num_targets)
    buf = kj[None, :] <= qi[:, None]
    tgt = kj[None, :] < (qi - num_targets)[:, None]
    m = torch.where((qi < num_targets)[:, None], buf, tgt)
    return m[None, None]


def merge_attention(out_a: Tensor, lse_a: Tensor, out_b: Tensor, lse_b: Tensor) -> Tensor:
    """Log-sum-exp merge of two partial attentions (triton_kernels.py:478-524)."""
    top = torch.maximum(lse_a, lse_b)
    wa = torch.exp(lse_a - top)
    wb = torch.exp(lse_b - top)
    tot = wa + wb
    wa = wa / tot
    wb = wb / tot
    return (wa.unsqueeze(-1) * out_a + wb.unsqueeze(-1) * out_b).to(out_a.dtype)


def hybrid_attention(q, k_ctx, v_ctx, k_buf, v_buf, buf_mask=None) -> Tensor:
    """Context + buffer attention merged (triton_kernels.py:705-755)."""
    out_c, lse_c = context_attention(q, k_ctx, v_ctx)
    if k_buf.shape[2] == 0:
        return out_c
    out_b, lse_b = buffer_attention(q, k_buf, v_buf, mask=buf_mask)
    return merge_attention(out_c, lse_c, out_b, lse_b)


def hybrid_teacher_forcing_attention(q, k_ctx, v_ctx, k_buf, v_buf, num_targets) -> Tensor:
    """Teacher-forcing variant (triton_kernels.py:662-702)."""
    if q.shape[2] != 2 * num_targets:
        raise ValueError("Expected 2*num_targets queries for teacher forcing.")
    if k_buf.shape[2] != num_targets:
        raise ValueError("Expected buffer length to match num_targets.")
    out_c, lse_c = context_attention(q, k_ctx, v_ctx)
    mask = teacher_forcing_buffer_mask(num_targets)
    out_b, lse_b = buffer_attention(q, k_buf, v_buf, mask=mask)
    return merge_attention(out_c, lse_c, out_b, lse_b)


def masked_attention(q: Tensor, k: Tensor, v: Tensor, mask: Optional[Tensor]) -> Tensor:
    """One-shot softmax attention over explicit K/V with a boolean mask.

    Second witness (the semantics of the reference's flex_attention calls,
    inference.py:622, 676, 735): q [B,H,Lq,Dh], k/v [B,H,Lk,Dh]."""
    scores = torch.matmul(q, k.transpose(-2, -1)) * (q.shape[-1] ** -0.5)
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(scores, dim=-1), v)


# --------------------------------------------------------------------------
# mixture-of-Gaussians head
# --------------------------------------------------------------------------

def head_params(sd: Dict[str, Tensor], z: Tensor):
    """mean, std, weight, log_weight each [..., K] (model.py:190-209, dim_y = 1)."""
    hid = gelu_erf(linear(z, sd["head.head.0.weight"], sd["head.head.0.bias"]))
    raw = linear(hid, sd["head.head.2.weight"], sd["head.head.2.bias"])
    K = sd["head.mean_bias"].numel()
    raw = raw.reshape(*raw.shape[:-1], K, 3)
    mean = raw[..., 0] + sd["head.mean_bias"]
    std = torch.nn.functional.softplus(raw[..., 1] + sd["head.std_bias"]).clamp(max=STD_MAX) + STD_MIN
    logw = torch.log_softmax(raw[..., 2] + sd["head.weight_bias"], dim=-1)
    return mean, std, logw.exp(), logw


def head_logpdf(mean, std, logw, y: Tensor) -> Tensor:
    """Mixture log density of y [...] (model.py:241-249)."""
    yy = y.unsqueeze(-1)
    lp = -0.5 * (math.log(2 * math.pi) + 2 * std.log() + ((yy - mean) / std) ** 2) + logw
    return torch.logsumexp(lp, dim=-1)


def head_sample(mean, std, weight, expo: Tensor, normal: Tensor) -> Tuple[Tensor, Tensor]:
    """Draw from the mixture with pre-drawn variates.

    ``torch.multinomial(w, 1)`` equals ``argmax(w / Exp(1))`` and is followed
    by one standard normal (model.py:251-266).  expo [..., K], normal [...]."""
    idx = (weight / expo).argmax(dim=-1, keepdim=True)
    m = torch.gather(mean, -1, idx).squeeze(-1)
    s = torch.gather(std, -1, idx).squeeze(-1)
    return m + s * normal, idx.squeeze(-1)


# --------------------------------------------------------------------------
# predictor
# --------------------------------------------------------------------------

@dataclass
class Emulation:
    """Where to round to bf16 to emulate the bf16 device mode on the CPU.

    qkv: round q, k, v after projection (tensor-core operands / KV cache);
    p:   round softmax numerators before the P.V product and K/V reads;
    act: round the activation entering every weight matmul;
    jitter: non-zero seed: instead of rounding, multiply q, k, v (and the softmax numerators when
         ``p`` is set) by 1 + d with d uniform in +-2^-9, the relative error bound of bf16
         rounding.  Several seeds give several realisations of the same rounding noise, which
         is how the tests estimate how strongly one target amplifies it."""
    qkv: bool = False
    p: bool = False
    act: bool = False
    jitter: int = 0


def layer_count(sd: Dict[str, Tensor]) -> int:
    n = 0
    while f"backbone.layers.{n}.norm1.weight" in sd:
        n += 1
    return n


class OraclePredictor:
    """CPU restatement of the reference predictor's shared-context backend.

    ``shared=True`` follows ``backend="triton_shared_context"`` (context of
    batch element 0 used for every stream, inference.py:191-193);
    ``shared=False`` gives every batch element its own context K/V, the
    semantics of ``backend="flex_attention"`` (inference.py:160-178, 423-453).
    """

    def __init__(self, sd: Dict[str, Tensor], n_heads: int, emu: Optional[Emulation] = None):
        self.sd = sd
        self.H = n_heads
        self.D = sd["embedder.x_embed.bias"].numel()
        self.Dh = self.D // n_heads
        self.L = layer_count(sd)
        self.S = sd["ar_tokens"].shape[0]
        self.emu = emu or Emulation()
        self.k_ctx = []
        self.v_ctx = []
        self.k_buf = []
        self.v_buf = []
        self._jit = torch.Generator().manual_seed(self.emu.jitter) if self.emu.jitter else None

    def _jitter(self, t: Tensor) -> Tensor:
        d = (torch.rand(t.shape, generator=self._jit, dtype=torch.float32) * 2.0 - 1.0) * 2.0 ** -9
        return t * (1.0 + d.to(t.dtype))

    # -- dense pieces ------------------------------------------------------
    def _a(self, x):
        return _bf16_round(x) if self.emu.act else x

    def _pre(self, l: int, x: Tensor):
        """x -> x1, q, k, v  (inference.py:771-783): the feature attention runs
        over a single token, so its softmax is 1 and it reduces to
        out_proj(v_proj(x))."""
        sd, p = self.sd, f"backbone.layers.{l}."
        f = linear(self._a(linear(self._a(x), sd[p + "attn_features.v_proj.weight"])),
                   sd[p + "attn_features.out_proj.weight"])
        x1 = layer_norm(f + x, sd[p + "norm1.weight"], sd[p + "norm1.bias"])
        xa = self._a(x1)
        q = linear(xa, sd[p + "attn_rows.q_proj.weight"])
        k = linear(xa, sd[p + "attn_rows.k_proj.weight"])
        v = linear(xa, sd[p + "attn_rows.v_proj.weight"])
        if self._jit is not None:
            q, k, v = self._jitter(q), self._jitter(k), self._jitter(v)
        elif self.emu.qkv:
            q, k, v = _bf16_round(q), _bf16_round(k), _bf16_round(v)
        return x1, q, k, v

    def _post(self, l: int, x1: Tensor, attn: Tensor) -> Tensor:
        """attention output -> layer output (inference.py:825-831)."""
        sd, p = self.sd, f"backbone.layers.{l}."
        x2 = layer_norm(x1 + linear(self._a(attn), sd[p + "attn_rows.out_proj.weight"]),
                        sd[p + "norm2.weight"], sd[p + "norm2.bias"])
        h = gelu_erf(linear(self._a(x2), sd[p + "ff.0.weight"], sd[p + "ff.0.bias"]))
        ff = linear(self._a(h), sd[p + "ff.2.weight"], sd[p + "ff.2.bias"])
        return layer_norm(x2 + ff, sd[p + "norm3.weight"], sd[p + "norm3.bias"])

    def _heads(self, t: Tensor) -> Tensor:
        """[B,N,D] -> [B,H,N,Dh]"""
        B, N, _ = t.shape
        return t.view(B, N, self.H, self.Dh).transpose(1, 2)

    def _unheads(self, t: Tensor) -> Tensor:
        B, H, N, Dh = t.shape
        return t.transpose(1, 2).reshape(B, N, H * Dh)

    def _softmax_pv(self, scores: Tensor, v: Tensor, dead: Optional[Tensor] = None) -> Tensor:
        p = torch.softmax(scores, dim=-1)
        if self.emu.p:
            # numerator rounded to bf16, denominator kept exact (fp32 row sum)
            top = scores.max(dim=-1, keepdim=True).values
            top = torch.where(torch.isinf(top), torch.zeros_like(top), top)
            e = torch.exp(scores - top)
            num = self._jitter(e) if self._jit is not None else _bf16_round(e)
            p = num / e.sum(dim=-1, keepdim=True).clamp_min(1e-38)
        if dead is not None:
            p = torch.where(dead.unsqueeze(-1), torch.zeros_like(p), p)
        return torch.matmul(p, v)

    def _attend(self, l: int, q: Tensor, k_buf: Optional[Tensor], v_buf: Optional[Tensor],
                buf_mask: Optional[Tensor] = None) -> Tensor:
        """Attention of q [B,H,Lq,Dh] over the layer's context K/V plus the
        given private buffer K/V [B,H,Nb,Dh] (None or Nb = 0: context only).

        Shared context: context part, buffer part and log-sum-exp merge, the
        structure of hybrid_attention (triton_kernels.py:705-755).  Per-batch
        context: one softmax over the concatenated keys (the flex_attention
        call of inference.py:735)."""
        scale = self.Dh ** -0.5
        kc, vc = self.k_ctx[l], self.v_ctx[l]
        has_buf = k_buf is not None and k_buf.shape[2] > 0
        if self.shared:
            sc = torch.matmul(q, kc.transpose(-2, -1)) * scale        # kc [1,H,Nc,Dh] broadcasts
            lse_c = torch.logsumexp(sc.float(), dim=-1)
            out_c = self._softmax_pv(sc, vc)
            if not has_buf:
                return out_c
            sb = torch.matmul(q, k_buf.transpose(-2, -1)) * scale
            dead = None
            if buf_mask is not None:
                sb = sb.masked_fill(~buf_mask, float("-inf"))
                dead = ~buf_mask.any(dim=-1)
            lse_b = torch.logsumexp(sb.float(), dim=-1)
            pb = torch.softmax(sb, dim=-1)
            if dead is not None:
                pb = torch.where(dead.unsqueeze(-1), torch.zeros_like(pb), pb)
            out_b = torch.matmul(pb, v_buf)
            return merge_attention(out_c, lse_c, out_b, lse_b)
        if not has_buf:
            return self._softmax_pv(torch.matmul(q, kc.transpose(-2, -1)) * scale, vc)
        kf, vf = torch.cat([kc, k_buf], dim=2), torch.cat([vc, v_buf], dim=2)
        sf = torch.matmul(q, kf.transpose(-2, -1)) * scale
        if buf_mask is not None:
            Nc = kc.shape[2]
            full = torch.cat([torch.ones(*buf_mask.shape[:-1], Nc, dtype=torch.bool), buf_mask], dim=-1)
            sf = sf.masked_fill(~full, float("-inf"))
        return self._softmax_pv(sf, vf)

    def final_norm(self, x):
        return layer_norm(x, self.sd["backbone.norm.weight"], self.sd["backbone.norm.bias"])

    # -- prefill -------------------------------------------------------------
    def prefill(self, xc: Tensor, yc: Tensor, shared: bool = True, q_chunk: int = 2048) -> None:
        """Populate the context K/V of every layer (inference.py:181-223,
        633-685).  The final backbone norm is not applied here."""
        if shared:
            xc, yc = xc[0:1], yc[0:1]
        x = embed_rows(self.sd, xc, yc, MARKER_CONTEXT)
        self.k_ctx, self.v_ctx = [], []
        self.shared = shared
        for l in range(self.L):
            x1, q, k, v = self._pre(l, x)
            qh, kh, vh = self._heads(q), self._heads(k), self._heads(v)
            self.k_ctx.append(kh)   # [G,H,Nc,Dh], G = 1 when shared
            self.v_ctx.append(vh)
            # query rows in chunks: a row's arithmetic does not depend on the chunking, and a
            # 16384-row context never materialises its 16384 x 16384 score matrix
            a = torch.cat([self._softmax_pv(torch.matmul(qh[:, :, c0:c0 + q_chunk], kh.transpose(-2, -1))
                                            * (self.Dh ** -0.5), vh)
                           for c0 in range(0, qh.shape[2], q_chunk)], dim=2)
            x = self._post(l, x1, self._unheads(a))
        self.k_buf = [None] * self.L
        self.v_buf = [None] * self.L
        self.buffer_len = 0

    # -- decode --------------------------------------------------------------
    def decode(self, emb: Tensor, commit: int) -> Tensor:
        """One step for N in {1,2} new tokens per stream (inference.py:226-276,
        746-833).  Token 0 of an N=2 step is the buffer token (appended to the
        private cache, sees context + all buffers including itself); the last
        token is the target (sees context + all buffers, never itself)."""
        B, N, _ = emb.shape
        if N not in (1, 2):
            raise ValueError("Shared-context decode only supports N=1 (target) or N=2 (buffer, target).")
        x = emb
        for l in range(self.L):
            x1, q, k, v = self._pre(l, x)
            qh, kh, vh = self._heads(q), self._heads(k), self._heads(v)
            if N == 2:
                kb, vb = kh[:, :, 0:1], vh[:, :, 0:1]
                if self.k_buf[l] is None:
                    kall, vall = kb, vb
                else:
                    kall = torch.cat([self.k_buf[l], kb], dim=2)
                    vall = torch.cat([self.v_buf[l], vb], dim=2)
                if commit:
                    self.k_buf[l], self.v_buf[l] = kall, vall
            else:
                kall, vall = self.k_buf[l], self.v_buf[l]
            a = self._attend(l, qh, kall, vall)
            x = self._post(l, x1, self._unheads(a))
        self.buffer_len += commit
        return self.final_norm(x)

    def sample_sequence(self, xc: Tensor, yc: Tensor, xt: Tensor, expo: Tensor, normal: Tensor,
                        shared: bool = True):
        """AR sampling (inference.py:323-366) with pre-drawn variates.

        expo [Nt,B,K] Exp(1) draws, normal [Nt,B] N(0,1) draws, in the order
        the reference consumes them.  Returns samples [B,Nt], the log density
        of each drawn value under the step's mixture [B,Nt], and the chosen
        components [B,Nt]."""
        B, Nt, _ = xt.shape
        self.prefill(xc, yc, shared=shared)
        ys, lds, comps = [], [], []
        prev_y = None
        for t in range(Nt):
            tgt = embed_rows(self.sd, xt[:, t:t + 1], None, MARKER_TARGET)
            if t == 0:
                emb, commit = tgt, 0
            else:
                ar = torch.full((B, 1), t % self.S, dtype=torch.long)
                buf = embed_rows(self.sd, xt[:, t - 1:t], prev_y, MARKER_BUFFER, ar)
                emb, commit = torch.cat([buf, tgt], dim=1), 1
            z = self.decode(emb, commit)[:, -1]
            mean, std, w, logw = head_params(self.sd, z)
            y, idx = head_sample(mean, std, w, expo[t], normal[t])
            ys.append(y)
            lds.append(head_logpdf(mean, std, logw, y))
            comps.append(idx)
            prev_y = y.unsqueeze(1)
        return torch.stack(ys, 1), torch.stack(lds, 1), torch.stack(comps, 1)

    # -- teacher forcing -------------------------------------------------------
    def evaluate_joint_density(self, xc, yc, xt, yt, shared: bool = True) -> Tensor:
        """Teacher-forced per-target log density [B,Nt] (inference.py:392-420,
        835-890).  New tokens are [Buffer_0..Buffer_{Nt-1}, Target_0..Target_{Nt-1}];
        buffer j carries (x_j, y_j) and AR token j mod S."""
        B, Nt, _ = xt.shape
        self.prefill(xc, yc, shared=shared)
        ar = (torch.arange(Nt) % self.S).unsqueeze(0).expand(B, -1)
        buf = embed_rows(self.sd, xt, yt, MARKER_BUFFER, ar)
        tgt = embed_rows(self.sd, xt, None, MARKER_TARGET)
        x = torch.cat([buf, tgt], dim=1)
        mask = teacher_forcing_buffer_mask(Nt)
        for l in range(self.L):
            x1, q, k, v = self._pre(l, x)
            qh, kh, vh = self._heads(q), self._heads(k), self._heads(v)
            a = self._attend(l, qh, kh[:, :, :Nt], vh[:, :, :Nt], buf_mask=mask)
            x = self._post(l, x1, self._unheads(a))
        z = self.final_norm(x)[:, Nt:]
        mean, std, w, logw = head_params(self.sd, z)
        return head_logpdf(mean, std, logw, yt)

    # -- masked forward (the training forward's row mask, inference only) -------
    def forward_masked(self, xc, yc, xb, yb, xt, yt, visible, shared: bool = False) -> Tensor:
        """Per-target log density [B,Nt] of the training forward (model.py:317-369)
        under a row mask of the create_row_mask family (attention.py:86-175):
        context rows see the context; the non-context rows
        [Buffer_0..Buffer_{Nb-1}, Target_0..Target_{Nt-1}] see the context plus the
        first ``visible[j]`` buffer rows.  Buffer j carries ar_tokens[j] (Nb <= S).
        Because no row is visible to a context row except context rows, the
        context part equals ``prefill`` and the rest is one pass over Nb + Nt
        tokens per dataset."""
        B, Nt, _ = xt.shape
        Nb = xb.shape[1]
        if Nb > self.S:
            raise ValueError("more buffer rows than AR position tokens")
        self.prefill(xc, yc, shared=shared)
        tgt = embed_rows(self.sd, xt, None, MARKER_TARGET)
        if Nb:
            ar = torch.arange(Nb).unsqueeze(0).expand(B, -1)
            x = torch.cat([embed_rows(self.sd, xb, yb, MARKER_BUFFER, ar), tgt], dim=1)
        else:
            x = tgt
        vis = torch.as_tensor(visible, dtype=torch.long).clamp(0, Nb)
        mask = (torch.arange(Nb)[None, :] < vis[:, None])[None, None]      # [1,1,Nb+Nt,Nb]
        for l in range(self.L):
            x1, q, k, v = self._pre(l, x)
            qh, kh, vh = self._heads(q), self._heads(k), self._heads(v)
            if Nb:
                a = self._attend(l, qh, kh[:, :, :Nb], vh[:, :, :Nb], buf_mask=mask)
            else:
                a = self._attend(l, qh, None, None)
            x = self._post(l, x1, self._unheads(a))
        z = self.final_norm(x)[:, Nb:]
        mean, std, w, logw = head_params(self.sd, z)
        return head_logpdf(mean, std, logw, yt)


def backbone_forward(sd: Dict[str, Tensor], n_heads: int, x: Tensor, n_ctx: int, n_buf: int, visible,
                     prefix: str = ""):
    """The backbone on inputs with C column tokens per row, x [B,R,C,D] -> [B,R,C,D]
    (model.py:100-147 of the reference): per layer feature attention across the C tokens of a row
    (dense), LayerNorm, row attention over the R rows of every column under a row mask of the
    create_row_mask family (rows [context | buffer | other]; non-context row j sees the context and
    the first visible[j] buffer rows; context rows see the context), LayerNorm, MLP, LayerNorm; the
    final LayerNorm at the end.  Also returns the row-attention K, V [B*C,H,R,Dh] of every layer."""
    B, R, C, D = x.shape
    H, Dh = n_heads, D // n_heads
    allowed = torch.zeros(R, R, dtype=torch.bool)
    allowed[:, :n_ctx] = True
    for j, v in enumerate(visible):
        allowed[n_ctx + j, n_ctx:n_ctx + int(v)] = True

    def mha(p, t, mask):
        G, S, _ = t.shape
        hd = lambda w: linear(t, sd[p + w]).view(G, S, H, Dh).transpose(1, 2)
        q, k, v = hd("q_proj.weight"), hd("k_proj.weight"), hd("v_proj.weight")
        o = masked_attention(q, k, v, mask)
        return linear(o.transpose(1, 2).reshape(G, S, D), sd[p + "out_proj.weight"]), (k, v)

    kvs = []
    L = 0
    while f"{prefix}layers.{L}.norm1.weight" in sd:
        L += 1
    for l in range(L):
        p = f"{prefix}layers.{l}."
        xf = x.reshape(B * R, C, D)
        a, _ = mha(p + "attn_features.", xf, None)
        x = layer_norm((a + xf).reshape(B, R, C, D), sd[p + "norm1.weight"], sd[p + "norm1.bias"])
        xr = x.permute(0, 2, 1, 3).reshape(B * C, R, D)
        a, kv = mha(p + "attn_rows.", xr, allowed)
        kvs.append(kv)
        x = layer_norm((a + xr).reshape(B, C, R, D).permute(0, 2, 1, 3), sd[p + "norm2.weight"], sd[p + "norm2.bias"])
        ff = linear(gelu_erf(linear(x, sd[p + "ff.0.weight"], sd[p + "ff.0.bias"])), sd[p + "ff.2.weight"], sd[p + "ff.2.bias"])
        x = layer_norm(x + ff, sd[p + "norm3.weight"], sd[p + "norm3.bias"])
    return layer_norm(x, sd[prefix + "norm.weight"], sd[prefix + "norm.bias"]), kvs


def row_mask_visible(n_buf: int, n_targets: int, attending_chunks: Optional[int] = None):
    """Visible-buffer counts of the non-context rows under create_row_mask
    (attention.py:86-175): buffer j sees buffers <= j; target t sees buffers
    <= t mod Nb while t < attending_chunks * Nb (default attending_chunks =
    Nt // (2 Nb)) and no buffer after that."""
    if attending_chunks is None:
        attending_chunks = n_targets // (2 * n_buf) if n_buf else 0
    vis = [j + 1 for j in range(n_buf)]
    for t in range(n_targets):
        vis.append((t % n_buf) + 1 if n_buf and t < attending_chunks * n_buf else 0)
    return vis


# --------------------------------------------------------------------------
# synthetic workloads (the benchmark configurations' generators)
# --------------------------------------------------------------------------

def make_dataset(seed: int, n_rows: int, n_feat: int, hidden: int = 32, noise: float = 0.1,
                 product_frac: float = 0.0):
    """x ~ N(0,1) iid standardised per column; y = tanh-MLP(F->h->h->1) with
    N(0, 1/fan_in) weights plus N(0, noise^2).  Optionally a fraction of the
    columns is replaced by pairwise products of two other columns."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_rows, n_feat, generator=g)
    n_prod = int(round(product_frac * n_feat))
    for j in range(n_prod):
        a = (2 * j + 1) % n_feat
        b = (2 * j + 2) % n_feat
        x[:, n_feat - 1 - j] = x[:, a] * x[:, b]
    x = (x - x.mean(0)) / x.std(0)
    w1 = torch.randn(n_feat, hidden, generator=g) / math.sqrt(n_feat)
    w2 = torch.randn(hidden, hidden, generator=g) / math.sqrt(hidden)
    w3 = torch.randn(hidden, 1, generator=g) / math.sqrt(hidden)
    y = (torch.tanh(torch.tanh(x @ w1) @ w2) @ w3)[:, 0]
    y = y + noise * torch.randn(n_rows, generator=g)
    return x, y


def draw_variates(seed: int, n_steps: int, batch: int, n_comp: int, dtype=torch.float32):
    """Exp(1) [Nt,B,K] and N(0,1) [Nt,B] in the reference's consumption order:
    per step one exponential fill of [B,K] (inside torch.multinomial) and then
    one normal fill of [B,1,1,1] (model.py:257, 265)."""
    g = torch.Generator().manual_seed(seed)
    ex, no = [], []
    for _ in range(n_steps):
        ex.append(torch.empty(batch, n_comp, dtype=dtype).exponential_(1.0, generator=g))
        no.append(torch.randn(batch, 1, 1, 1, generator=g, dtype=dtype).view(batch))
    return torch.stack(ex), torch.stack(no)
