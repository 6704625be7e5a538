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


def _split_bf16(w: torch.Tensor):
    """fp64 matrix -> (hi, lo) bf16 parts with hi + lo ~= w to 16 mantissa bits."""
    hi = w.to(torch.float32).to(torch.bfloat16)
    lo = (w - hi.to(torch.float64)).to(torch.float32).to(torch.bfloat16)
    return hi, lo


def _swizzle_block(blk: torch.Tensor) -> torch.Tensor:
    """[rows][64] bf16 -> the 128-byte-swizzled K-major shared-memory image of that block:
    16-byte chunk c of row r is stored at chunk position c ^ (r % 8)."""
    rows = blk.shape[0]
    chunks = blk.reshape(rows, 8, 8)
    pos = torch.arange(8, device=blk.device)[None, :] ^ (torch.arange(rows, device=blk.device)[:, None] % 8)
    out = torch.empty_like(chunks)
    out.scatter_(1, pos[:, :, None].expand(rows, 8, 8), chunks)
    return out.reshape(-1)


def tile_weight(w: torch.Tensor, mode: str, force_lo: bool = False):
    """Tile an nn.Linear weight [N][K] (fp64) for the tensor-core chain.

    The result is the exact byte stream the kernel's weight ring consumes: a sequence of
    slabs, each a stack of swizzled [rows][64 k] blocks, hi part then (optionally) lo part.
      mode "full":   one slab per 64-wide k-chunk holding all N rows            (N = d_model)
      mode "ntile":  per 128-row output tile one 16 KB slab per k-chunk         (hidden GEMMs)
    Returns (flat bf16 tensor, has_lo)."""
    N, K = w.shape
    assert K % 64 == 0
    hi, lo = _split_bf16(w)
    has_lo = force_lo or bool((lo != 0).any())
    slabs = []
    if mode == "full":
        for kc in range(K // 64):
            for part in ((hi, lo) if has_lo else (hi,)):
                slabs.append(_swizzle_block(part[:, kc * 64:(kc + 1) * 64].contiguous()))
    else:
        assert N % 128 == 0
        for j in range(N // 128):
            for part in ((hi, lo) if has_lo else (hi,)):
                for kc in range(K // 64):
                    slabs.append(_swizzle_block(part[j * 128:(j + 1) * 128, kc * 64:(kc + 1) * 64].contiguous()))
    return torch.cat(slabs), has_lo


class PackedModel:
    """All packing arithmetic (transposes, the fold of the feature attention, hi / lo splits,
    swizzled tiles) runs on the host in fp64, once per model version; the device sees two copies
    (the fp32 buffer and the bf16 tile stream) and no packing kernels."""

    def __init__(self, embedder, backbone, head, ar_tokens, device: torch.device):
        target, device = device, torch.device("cpu")
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
        flat = flat.to(target)
        self.flat = flat
        base = flat.data_ptr()

        def P(name):
            return C.c_void_p(base + 4 * offsets[name])

        self._layers = (_lib.LayerWeights * self.n_layers)()
        for i in range(self.n_layers):
            for f, _ in _lib.LayerWeights._fields_:
                if not f.startswith("tc_"):
                    setattr(self._layers[i], f, P(f"{i}.{f}"))
        m = _lib.Model()
        m.d_model, m.n_heads, m.head_dim, m.d_ff = self.d_model, self.n_heads, self.head_dim, self.d_ff
        m.n_layers, m.n_comp, m.n_ar_tokens = self.n_layers, self.n_comp, self.n_ar
        for f in ("wx", "bx", "wy", "by", "marker", "ar_tokens", "lnf_g", "lnf_b", "wa_t", "ba", "wb_t", "bb",
                  "mean_bias", "std_bias", "weight_bias"):
            setattr(m, f, P(f))
        m.layers = C.cast(self._layers, C.POINTER(_lib.LayerWeights))
        self.struct = m
        self._pack_tensor_core(embedder, backbone, head, target)

    def _pack_tensor_core(self, embedder, backbone, head, target):
        """bf16 hi/lo tiles for the tcgen05 per-token chain (d_model in {64,128,192}, d_ff % 128 == 0,
        3K <= 16).  Other shapes keep the fp32 FMA chain (the tc_* pointers stay NULL)."""
        D, Dff = self.d_model, self.d_ff
        device = torch.device("cpu")
        self.tc_flat = None
        if D not in (64, 128, 192) or Dff % 128 != 0 or Dff > 1024 or 3 * self.n_comp > 16:
            return
        f64 = lambda t: t.detach().to(device=device, dtype=torch.float64)
        items = []

        def add(name, w, mode, force_lo=False):
            flat, has_lo = tile_weight(w, mode, force_lo)
            items.append((name, flat))
            return has_lo

        layer_lo = []
        for i, l in enumerate(backbone.layers):
            r = l.attn_rows
            bits = 0
            bits |= 1 * add(f"{i}.tc_wo", f64(r.out_proj.weight), "full")
            bits |= 2 * add(f"{i}.tc_w1", f64(l.ff[0].weight), "ntile")
            bits |= 4 * add(f"{i}.tc_w2", f64(l.ff[2].weight), "full")
            wf = f64(l.attn_features.out_proj.weight) @ f64(l.attn_features.v_proj.weight)
            bits |= 8 * add(f"{i}.tc_wf", wf, "full")
            # q, k, v must agree on the lo part: they share one flag
            qkv_lo = any(bool((_split_bf16(f64(p.weight))[1] != 0).any()) for p in (r.q_proj, r.k_proj, r.v_proj))
            for nm, p in (("q", r.q_proj), ("k", r.k_proj), ("v", r.v_proj)):
                add(f"{i}.tc_w{nm}", f64(p.weight), "full", force_lo=qkv_lo)
            bits |= 16 * qkv_lo
            layer_lo.append(bits)
        head_bits = 1 * add("tc_wa", f64(head.head[0].weight), "ntile")
        wb = torch.zeros(16, Dff, dtype=torch.float64, device=device)
        wb[: 3 * self.n_comp] = f64(head.head[2].weight)
        head_bits |= 2 * add("tc_wb", wb, "full")
        offs, tot = {}, 0
        for name, t in items:
            offs[name] = tot
            tot += (t.numel() + 511) // 512 * 512          # 1 KiB alignment of every matrix
        flat = torch.zeros(tot, dtype=torch.bfloat16, device=device)
        for name, t in items:
            flat[offs[name]:offs[name] + t.numel()] = t
        flat = flat.to(target)
        self.tc_flat = flat
        base = flat.data_ptr()
        for i in range(self.n_layers):
            lw = self._layers[i]
            lw.tc_wo = base + 2 * offs[f"{i}.tc_wo"]
            lw.tc_w1 = base + 2 * offs[f"{i}.tc_w1"]
            lw.tc_w2 = base + 2 * offs[f"{i}.tc_w2"]
            lw.tc_wf = base + 2 * offs[f"{i}.tc_wf"]
            lw.tc_wqkv = base + 2 * offs[f"{i}.tc_wq"]
            lw.tc_lo = layer_lo[i]
        self.struct.tc_wa = base + 2 * offs["tc_wa"]
        self.struct.tc_wb = base + 2 * offs["tc_wb"]
        self.struct.tc_head_lo = head_bits

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
