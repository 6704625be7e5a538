"""Model classes of the drop-in package.

Same constructors, attribute names, default initialisation and state_dict keys
as the reference (ar_tabpfn/model/model.py:23-315), so that a trained reference
checkpoint loads with ``load_state_dict``.  The embedder and the mixture head
run as CUDA kernels through the C ABI; the training forward is not part of this
build.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor, nn

from .. import _lib
from .attention import MultiheadAttention


def _f32(t: Tensor) -> Tensor:
    return t.detach().to(torch.float32).contiguous()


class _EmbedWeights:
    """Minimal artab_model view holding only what artab_embed reads."""

    def __init__(self, emb: "Embedder", device):
        D = emb.x_embed.bias.numel()
        flat = torch.cat([_f32(emb.x_embed.weight[:, 0]), _f32(emb.x_embed.bias), _f32(emb.y_embed.weight[:, 0]),
                          _f32(emb.y_embed.bias), _f32(emb.marker_embed.weight).reshape(-1)]).to(device)
        self.flat = flat
        m = _lib.Model()
        m.d_model, m.n_ar_tokens = D, 0
        base = flat.data_ptr()
        for i, f in enumerate(("wx", "bx", "wy", "by", "marker")):
            setattr(m, f, base + 4 * D * i)
        self.struct = m


class Embedder(nn.Module):
    """(x, y) rows -> D-dim tokens plus a marker for context / buffer / target
    (reference: ar_tabpfn/model/model.py:23-76)."""

    def __init__(self, d_model: int):
        super().__init__()
        self.x_embed = nn.Linear(1, d_model)
        self.y_embed = nn.Linear(1, d_model)
        self.marker_embed = nn.Embedding(3, d_model)
        self._marker_lookup = {"target": 0, "context": 1, "buffer": 2}

    def _embed(self, x: Tensor, y: Optional[Tensor], kind: str) -> Tensor:
        lib = _lib.lib()
        B, N, F = x.shape
        dev = x.device
        key = (str(dev),) + tuple((p.data_ptr(), p._version) for p in self.parameters())
        cached = getattr(self, "_artab_w", None)
        if cached is None or cached[0] != key:
            cached = (key, _EmbedWeights(self, dev))
            self._artab_w = cached
        w = cached[1]
        xf = _f32(x).reshape(B * N, F)
        yf = None
        if y is not None:
            yf = _f32(y).reshape(B * N)
        out = torch.empty(B * N, w.struct.d_model, device=dev, dtype=torch.float32)
        import ctypes as C
        _lib.check(lib.artab_embed(C.byref(w.struct), _lib.ptr(xf), _lib.ptr(yf), None, B * N, F,
                                   self._marker_lookup[kind], _lib.ptr(out), _lib.stream_ptr()))
        return out.view(B, N, -1).to(x.dtype)

    def embed_context(self, x: Tensor, y: Tensor) -> Tensor:
        """x [B,N,C], y [B,N] or [B,N,1] -> [B,N,D]"""
        return self._embed(x, y, "context")

    def embed_buffer(self, x: Tensor, y: Tensor) -> Tensor:
        """Buffer rows; the AR position token is added by the caller."""
        return self._embed(x, y, "buffer")

    def embed_target(self, x: Tensor) -> Tensor:
        return self._embed(x, None, "target")


class TwoStageTransformerLayer(nn.Module):
    """Feature attention + row attention + MLP, three post-norms
    (reference: ar_tabpfn/model/model.py:79-126)."""

    def __init__(self, d_model: int, n_heads: int, d_ff: int):
        super().__init__()
        self.attn_features = MultiheadAttention(d_model, n_heads)
        self.attn_rows = MultiheadAttention(d_model, n_heads)
        self.ff = nn.Sequential(nn.Linear(d_model, d_ff), nn.GELU(), nn.Linear(d_ff, d_model))
        self.norm1 = nn.LayerNorm(d_model)
        self.norm2 = nn.LayerNorm(d_model)
        self.norm3 = nn.LayerNorm(d_model)

    @torch.no_grad()
    def forward(self, x: Tensor, mask_features, mask_rows):
        """The reference's layer call (model.py:100-126) for inference, with ANY number of column
        tokens: x [B,R,C,D] -> (x [B,R,C,D], (K, V) of the row attention [B*C,H,R,Dh]).  Feature
        attention across the C tokens of a row under ``mask_features`` (a ``DenseMask``), row attention
        over the R rows of every column under ``mask_rows`` (a ``RowMask``); both softmax attentions
        run on this library's kernels, projections / LayerNorm / MLP are library calls.  The
        predictor's hot path (one token per row) does not come through here."""
        B, R, C, D = x.shape
        x_feat = x.reshape(B * R, C, D)
        attn_out, _ = self.attn_features(x_feat, x_feat, x_feat, mask_features)
        x = self.norm1((attn_out + x_feat).reshape(B, R, C, D))
        x_row = x.permute(0, 2, 1, 3).reshape(B * C, R, D)
        attn_out, kv = self.attn_rows(x_row, x_row, x_row, mask_rows)
        x = self.norm2((attn_out + x_row).reshape(B, C, R, D).permute(0, 2, 1, 3))
        return self.norm3(x + self.ff(x)), kv


class TwoStageTransformer(nn.Module):
    def __init__(self, d_model: int, n_heads: int, n_layers: int, d_ff: int):
        super().__init__()
        self.d_model = d_model
        self.layers = nn.ModuleList([TwoStageTransformerLayer(d_model, n_heads, d_ff) for _ in range(n_layers)])
        self.norm = nn.LayerNorm(d_model)

    @torch.no_grad()
    def forward(self, x: Tensor, mask_features, mask_rows):
        """x [B,R,C,D] through every layer and the final norm; returns (x, [(K, V) per layer]) like the
        reference (model.py:139-147).  Inference only."""
        kv_cache = []
        for layer in self.layers:
            x, kv = layer(x, mask_features, mask_rows)
            kv_cache.append(kv)
        return self.norm(x), kv_cache


class _HeadWeights:
    def __init__(self, head: "MixtureGaussianHead", device):
        lin0, lin2 = head.head[0], head.head[2]
        D, Dff, K = lin0.weight.shape[1], lin0.weight.shape[0], head.num_components
        parts = [_f32(lin0.weight).t().contiguous().reshape(-1), _f32(lin0.bias),
                 _f32(lin2.weight).t().contiguous().reshape(-1), _f32(lin2.bias),
                 _f32(head.mean_bias), _f32(head.std_bias), _f32(head.weight_bias)]
        offs, tot = [], 0
        for p in parts:
            offs.append(tot)
            tot += (p.numel() + 63) // 64 * 64
        flat = torch.zeros(tot, dtype=torch.float32, device=device)
        for o, p in zip(offs, parts):
            flat[o:o + p.numel()] = p.to(device)
        self.flat = flat
        m = _lib.Model()
        m.d_model, m.d_ff, m.n_comp = D, Dff, K
        for o, f in zip(offs, ("wa_t", "ba", "wb_t", "bb", "mean_bias", "std_bias", "weight_bias")):
            setattr(m, f, flat.data_ptr() + 4 * o)
        self.struct = m


class MixtureGaussianHead(nn.Module):
    """K-component Gaussian mixture over a scalar y
    (reference: ar_tabpfn/model/model.py:150-272)."""

    def __init__(self, d_model: int, d_ff: int, dim_y: int = 1, num_components: int = 5, std_min: float = 1e-3):
        super().__init__()
        if dim_y != 1:
            raise ValueError("this build supports dim_y = 1")
        self.dim_y = dim_y
        self.num_components = num_components
        self.std_min = std_min
        self.head = nn.Sequential(nn.Linear(d_model, d_ff), nn.GELU(), nn.Linear(d_ff, num_components * dim_y * 3))
        self.mean_bias = nn.Parameter(torch.linspace(-1.0, 1.0, num_components))
        delta = 1.0 / (num_components - 1)
        self.std_bias = nn.Parameter(torch.ones(num_components) * self._inv_softplus(delta))
        self.weight_bias = nn.Parameter(torch.zeros(num_components))

    @staticmethod
    def _inv_softplus(y: float) -> float:
        return math.log(math.exp(y) - 1)

    def _weights(self, device) -> _HeadWeights:
        key = (str(device),) + tuple((p.data_ptr(), p._version) for p in self.parameters())
        cached = getattr(self, "_artab_w", None)
        if cached is None or cached[0] != key:
            cached = (key, _HeadWeights(self, device))
            self._artab_w = cached
        return cached[1]

    def sample(self, z: Tensor, num_samples: int = 1) -> Tensor:
        """z [B,T,D] -> [B,T,num_samples,1].  With num_samples = 1 (what the sampler uses) torch's
        generator is consumed exactly like the reference: one Exp(1) fill of [B*T,K] (inside
        torch.multinomial) followed by one N(0,1) fill of [B,T,1,1].  num_samples > 1 draws the
        samples one after the other in that same pattern: the distribution is the reference's
        (model.py:251-266), the random stream is not (the reference's multinomial takes another
        route for several samples)."""
        if num_samples < 1:
            raise ValueError("num_samples must be >= 1")
        if num_samples > 1:
            return torch.cat([self.sample(z, 1) for _ in range(num_samples)], dim=2)
        import ctypes as C
        lib = _lib.lib()
        B, T, D = z.shape
        w = self._weights(z.device)
        zf = _f32(z).reshape(B * T, D)
        expo = torch.empty(B * T, self.num_components, device=z.device, dtype=z.dtype).exponential_(1)
        normal = torch.randn(B, T, 1, 1, device=z.device, dtype=z.dtype)
        y = torch.empty(B * T, device=z.device, dtype=torch.float32)
        # fp32 copies stay referenced until the launch is queued: a temporary released earlier could
        # hand its memory to the next conversion before the kernel has read it
        expo32, normal32 = _f32(expo), _f32(normal).reshape(-1)
        _lib.check(lib.artab_head_sample(C.byref(w.struct), _lib.ptr(zf), _lib.ptr(expo32),
                                         _lib.ptr(normal32), B * T, _lib.ptr(y), None, None,
                                         _lib.stream_ptr()))
        return y.view(B, T, 1, 1).to(z.dtype)

    def log_likelihood(self, z: Tensor, y: Tensor) -> Tensor:
        """z [B,T,D], y [B,T,1] -> [B,T]"""
        import ctypes as C
        lib = _lib.lib()
        B, T, D = z.shape
        w = self._weights(z.device)
        zf = _f32(z).reshape(B * T, D)
        yf = _f32(y).reshape(B * T)
        ld = torch.empty(B * T, device=z.device, dtype=torch.float32)
        _lib.check(lib.artab_head_logpdf(C.byref(w.struct), _lib.ptr(zf), _lib.ptr(yf), B * T, _lib.ptr(ld),
                                         _lib.stream_ptr()))
        return ld.view(B, T).to(z.dtype)

    def forward(self, *args, **kwargs):
        raise NotImplementedError("training loss is outside this build; use log_likelihood / sample")


class ARTabPFN(nn.Module):
    """Container with the reference's constructor and state_dict layout
    (reference: ar_tabpfn/model/model.py:275-315)."""

    def __init__(self, d_model: int = 128, n_heads: int = 4, n_layers: int = 6, d_ff: int = 256,
                 num_features: int = 10, buffer_size: int = 8, num_components: int = 5):
        super().__init__()
        self.d_model = d_model
        self.num_features = num_features
        self.buffer_size = buffer_size
        self.embedder = Embedder(d_model)
        self.backbone = TwoStageTransformer(d_model, n_heads, n_layers, d_ff)
        self.head = MixtureGaussianHead(d_model, d_ff, dim_y=1, num_components=num_components)
        self.ar_tokens = nn.Parameter(torch.randn(buffer_size, d_model) * 0.02)

    @classmethod
    def from_checkpoint(cls, path_or_dict, n_heads: int, num_features: int = 10, map_location="cpu") -> "ARTabPFN":
        """Build a model from a checkpoint of the reference's training script
        (``torch.save({"step": ..., "model": model.state_dict()})``, train.py:340-342) or from a
        plain state_dict.  The training script compiles ``embedder`` and ``head``, which prefixes
        their keys with ``_orig_mod.``; the prefix is removed.  Every size but the head count
        (not recoverable from the weights) and ``num_features`` (no weight depends on it) is read
        from the tensor shapes."""
        ck = torch.load(path_or_dict, map_location=map_location, weights_only=True) \
            if isinstance(path_or_dict, (str, bytes)) or hasattr(path_or_dict, "__fspath__") else path_or_dict
        sd = ck["model"] if isinstance(ck, dict) and "model" in ck and isinstance(ck["model"], dict) else ck
        sd = {k.replace("_orig_mod.", ""): v for k, v in sd.items()}
        S, D = sd["ar_tokens"].shape
        L = 0
        while f"backbone.layers.{L}.norm1.weight" in sd:
            L += 1
        if L == 0 or D % n_heads:
            raise ValueError("checkpoint has no transformer layers or d_model is not divisible by n_heads")
        m = cls(d_model=D, n_heads=n_heads, n_layers=L, d_ff=sd["backbone.layers.0.ff.0.weight"].shape[0],
                num_features=num_features, buffer_size=S, num_components=sd["head.mean_bias"].numel())
        m.load_state_dict(sd)
        return m.eval()

    @torch.no_grad()
    def forward(self, x_context: Tensor, y_context: Tensor, x_buffer: Tensor, y_buffer: Tensor,
                x_target: Tensor, mask_features, mask_rows, y_target: Optional[Tensor] = None):
        """The reference's forward (model.py:317-369) for inference: returns the loss
        ``-mean(log density of y_target)`` under ``mask_rows`` (a ``RowMask`` from
        ``create_row_mask``), or None without ``y_target``, like the reference.  No autograd
        graph is built: gradients, and with them training, are outside this build.  The
        per-target log densities of the call are kept in ``last_logdens`` [B,Nt]."""
        from .attention import RowMask
        from .inference import ARTabPFNPredictor
        if not isinstance(mask_rows, RowMask):
            raise TypeError("mask_rows must be the RowMask returned by create_row_mask (flex BlockMasks are "
                            "not decoded)")
        Nc, Nb, Nt = x_context.size(1), x_buffer.size(1), x_target.size(1)
        if (mask_rows.context_len, mask_rows.buffer_len, mask_rows.num_rows) != (Nc, Nb, Nc + Nb + Nt):
            raise ValueError("mask_rows was built for other row counts")
        if y_target is None:
            return None
        if y_target.dim() == 3:
            y_target = y_target[..., 0]
        pred = getattr(self, "_artab_fwd", None)
        if pred is None:
            pred = ARTabPFNPredictor.from_trained_model(self, backend="flex_attention")
            object.__setattr__(self, "_artab_fwd", pred)
        ld = pred.forward_masked(x_context, y_context, x_buffer, y_buffer, x_target, y_target, mask_rows.visible)
        object.__setattr__(self, "last_logdens", ld)
        return -ld.sum() / ld.numel()
