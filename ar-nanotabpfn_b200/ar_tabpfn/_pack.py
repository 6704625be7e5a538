"""Pack module weights into the flat fp32 device buffer the kernels read.

All matrices are stored transposed ([in][out]); the feature-attention pair
(out_proj, v_proj) is folded into one [D][D] matrix because that attention runs
over a single token (ar_tabpfn/model/inference.py:771-773 of the reference:
softmax over one key is 1, so the block equals out_proj(v_proj(x)) and the q/k
projections never influence the result).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import torch

from . import _lib

_ALIGN = 64  # floats


class PackedModel:
    def __init__(self, embedder, backbone, head, ar_tokens, device: torch.device):
        layers = list(backbone.layers)
        attn0 = layers[0].attn_rows
        self.d_model = int(backbone.norm.weight.numel())
        self.n_heads = int(attn0.n_heads)
        self.head_dim = int(attn0.head_dim)
        self.d_ff = int(layers[0].ff[0].weight.shape[0])
        self.n_layers = len(layers)
        self.n_comp = int(head.num_components)
        self.n_ar = int(ar_tokens.shape[0])
        if int(head.dim_y) != 1:
            raise ValueError("only dim_y = 1 is supported")
        if int(head.head[0].weight.shape[0]) != self.d_ff:
            raise ValueError("head hidden width must equal d_ff")

        items: List[Tuple[str, torch.Tensor]] = []

        def add(name, t):
            items.append((name, t.detach().to(device=device, dtype=torch.float64).contiguous()))

        def T(w):  # nn.Linear weight [out][in] -> [in][out]
            return w.detach().to(device=device, dtype=torch.float64).t().contiguous()

        e = embedder
        add("wx", e.x_embed.weight[:, 0]); add("bx", e.x_embed.bias)
        add("wy", e.y_embed.weight[:, 0]); add("by", e.y_embed.bias)
        add("marker", e.marker_embed.weight); add("ar_tokens", ar_tokens)
        add("lnf_g", backbone.norm.weight); add("lnf_b", backbone.norm.bias)
        add("wa_t", T(head.head[0].weight)); add("ba", head.head[0].bias)
        add("wb_t", T(head.head[2].weight)); add("bb", head.head[2].bias)
        add("mean_bias", head.mean_bias); add("std_bias", head.std_bias); add("weight_bias", head.weight_bias)
        for i, l in enumerate(layers):
            wv = l.attn_features.v_proj.weight.detach().to(device=device, dtype=torch.float64)
            wo = l.attn_features.out_proj.weight.detach().to(device=device, dtype=torch.float64)
            add(f"{i}.wf_t", (wo @ wv).t())
            add(f"{i}.ln1_g", l.norm1.weight); add(f"{i}.ln1_b", l.norm1.bias)
            r = l.attn_rows
            add(f"{i}.wqkv_t", torch.cat([T(r.q_proj.weight), T(r.k_proj.weight), T(r.v_proj.weight)], dim=1))
            add(f"{i}.wo_t", T(r.out_proj.weight))
            add(f"{i}.ln2_g", l.norm2.weight); add(f"{i}.ln2_b", l.norm2.bias)
            add(f"{i}.w1_t", T(l.ff[0].weight)); add(f"{i}.b1", l.ff[0].bias)
            add(f"{i}.w2_t", T(l.ff[2].weight)); add(f"{i}.b2", l.ff[2].bias)
            add(f"{i}.ln3_g", l.norm3.weight); add(f"{i}.ln3_b", l.norm3.bias)

        offsets, total = {}, 0
        for name, t in items:
            offsets[name] = total
            total += (t.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        flat = torch.zeros(total, dtype=torch.float32, device=device)
        for name, t in items:
            flat[offsets[name]:offsets[name] + t.numel()] = t.reshape(-1).to(torch.float32)
        self.flat = flat
        base = flat.data_ptr()

        def P(name):
            return C.c_void_p(base + 4 * offsets[name])

        self._layers = (_lib.LayerWeights * self.n_layers)()
        for i in range(self.n_layers):
            for f, _ in _lib.LayerWeights._fields_:
                setattr(self._layers[i], f, P(f"{i}.{f}"))
        m = _lib.Model()
        m.d_model, m.n_heads, m.head_dim, m.d_ff = self.d_model, self.n_heads, self.head_dim, self.d_ff
        m.n_layers, m.n_comp, m.n_ar_tokens = self.n_layers, self.n_comp, self.n_ar
        for f in ("wx", "bx", "wy", "by", "marker", "ar_tokens", "lnf_g", "lnf_b", "wa_t", "ba", "wb_t", "bb",
                  "mean_bias", "std_bias", "weight_bias"):
            setattr(m, f, P(f))
        m.layers = C.cast(self._layers, C.POINTER(_lib.LayerWeights))
        self.struct = m

    @property
    def ref(self):
        return C.byref(self.struct)


def packed_for(owner, embedder, backbone, head, ar_tokens, device) -> PackedModel:
    """Cache the packed weights on `owner`, keyed by device and parameter versions."""
    params = [ar_tokens] + list(embedder.parameters()) + list(backbone.parameters()) + list(head.parameters())
    key = (str(device),) + tuple((p.data_ptr(), p._version) for p in params)
    cached = getattr(owner, "_artab_packed", None)
    if cached is None or cached[0] != key:
        cached = (key, PackedModel(embedder, backbone, head, ar_tokens, device))
        owner._artab_packed = cached
    return cached[1]
