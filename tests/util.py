"""Shared helpers for the test-suite."""
import os

import torch

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load_golden(name):
    return torch.load(os.path.join(GOLD, name), weights_only=False)


def build_model(fx, device="cuda", bf16_round=False):
    """Shipped-package model carrying the fixture's weights."""
    import ar_tabpfn
    m = ar_tabpfn.ARTabPFN(**fx["cfg"]).eval()
    sd = fx["state_dict"]
    if bf16_round:
        sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    m.load_state_dict(sd)
    for p in m.parameters():
        p.requires_grad_(False)
    return m.to(device), sd


def ref_attention(q, k, v, mask=None):
    """Plain fp32 softmax attention (torch), q [B,H,Lq,Dh], k/v [B,H,Lk,Dh]."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * q.shape[-1] ** -0.5
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v.float()), torch.logsumexp(s, dim=-1)


def reference_kernels():
    """The reference's own ``ar_tabpfn.model.triton_kernels`` module, when the unmodified reference
    package is installed under ``baseline/_ref`` (imported under the alias ``ref_ar_tabpfn`` so that it
    cannot collide with the shipped package of the same name); None otherwise."""
    import importlib
    import sys
    import types
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "ar_tabpfn")
    if not os.path.isdir(root):
        return None
    if "ref_ar_tabpfn" not in sys.modules:
        pkg = types.ModuleType("ref_ar_tabpfn")
        pkg.__path__ = [root]
        sys.modules["ref_ar_tabpfn"] = pkg
    try:
        return importlib.import_module("ref_ar_tabpfn.model.triton_kernels")
    except Exception:  # noqa: BLE001  (a foreign package that does not import is the same as an absent one)
        return None
