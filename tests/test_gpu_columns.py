"""Several column tokens per row (C > 1): the backbone's module-level forward, whose feature
attention runs across the C tokens of a row and whose row attention runs over the rows of every
column, against golden outputs of the reference's own TwoStageTransformer and against the oracle."""
import pytest
import torch

import artab_oracle as orc
from util import load_golden

pytestmark = pytest.mark.gpu


def _backbone(c, dtype=torch.float32):
    from ar_tabpfn.model import TwoStageTransformer
    m = TwoStageTransformer(**c["cfg"]).eval()
    m.load_state_dict(c["state_dict"])
    return m.cuda().to(dtype)


def _masks(c):
    from ar_tabpfn.model import create_dense_mask, create_row_mask
    R = c["Nc"] + c["Nb"] + c["Nt"]
    return create_dense_mask(c["C"]), create_row_mask(R, context_len=c["Nc"], buffer_len=c["Nb"],
                                                       attending_chunks=c["attending_chunks"])


def test_backbone_with_column_tokens_fp32_golden():
    for c in load_golden("columns.pt"):
        m = _backbone(c)
        mf, mr = _masks(c)
        out, kvs = m(c["x"].cuda(), mf, mr)
        assert out.shape == c["out"].shape and len(kvs) == c["cfg"]["n_layers"]
        torch.testing.assert_close(out.cpu(), c["out"], atol=2e-5, rtol=1e-5)
        torch.testing.assert_close(kvs[0][0].cpu(), c["k0"], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(kvs[0][1].cpu(), c["v0"], atol=1e-5, rtol=1e-5)


def test_backbone_with_column_tokens_bf16():
    """bf16 tensors select the bf16 kernels (tensor cores at head_dim 32); compared with the fp32
    oracle on the same bf16-representable weights and inputs."""
    for c in load_golden("columns.pt"):
        sd = {k: v.to(torch.bfloat16).float() for k, v in c["state_dict"].items()}
        x = c["x"].to(torch.bfloat16).float()
        vis = orc.row_mask_visible(c["Nb"], c["Nt"], c["attending_chunks"])
        want, _ = orc.backbone_forward(sd, c["cfg"]["n_heads"], x, c["Nc"], c["Nb"], vis)
        m = _backbone(dict(c, state_dict=sd), torch.bfloat16)
        mf, mr = _masks(c)
        out, _ = m(x.cuda().to(torch.bfloat16), mf, mr)
        assert out.dtype == torch.bfloat16
        rel = float((out.float().cpu() - want).norm() / want.norm())
        assert rel <= 2e-2, rel   # the whole forward in bf16 tensors (library LayerNorm / GEMMs included)


def test_attention_module_matches_oracle_and_refuses_foreign_masks():
    from ar_tabpfn.model import MultiheadAttention, create_dense_mask
    torch.manual_seed(0)
    att = MultiheadAttention(64, 2).eval().cuda()
    x = torch.randn(5, 7, 64, device="cuda")
    out, (k, v) = att(x, x, x, create_dense_mask(7))
    sd = {n: p.detach().cpu() for n, p in att.state_dict().items()}
    hd = lambda w: orc.linear(x.cpu(), sd[w]).view(5, 7, 2, 32).transpose(1, 2)
    want = orc.masked_attention(hd("q_proj.weight"), hd("k_proj.weight"), hd("v_proj.weight"), None)
    want = orc.linear(want.transpose(1, 2).reshape(5, 7, 64), sd["out_proj.weight"])
    torch.testing.assert_close(out.cpu(), want, atol=1e-5, rtol=1e-5)
    assert k.shape == (5, 2, 7, 32) and v.shape == (5, 2, 7, 32)
    with pytest.raises(TypeError):
        att(x, x, x, object())
