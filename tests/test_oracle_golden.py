"""The CPU oracle against golden vectors produced by the real reference.

The fixtures under tests/golden were written by tests/golden/make_golden.py,
which imports the reference implementation; these tests pin the oracle to it.
"""
import os

import pytest
import torch

import artab_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return torch.load(os.path.join(GOLD, name), weights_only=False)


@pytest.fixture(scope="module")
def ops():
    return load("ops.pt")


def test_context_attention(ops):
    for c in ops["attn"]:
        out, lse = orc.context_attention(c["q"], c["k_ctx"], c["v_ctx"])
        torch.testing.assert_close(out, c["out_ctx"], atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(lse, c["lse_ctx"], atol=1e-6, rtol=1e-6)


def test_buffer_attention_and_merge(ops):
    for c in ops["attn"]:
        if c["k_buf"].shape[2] == 0:
            continue
        out, lse = orc.buffer_attention(c["q"], c["k_buf"], c["v_buf"])
        torch.testing.assert_close(out, c["out_buf"], atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(lse, c["lse_buf"], atol=1e-6, rtol=1e-6)
        merged = orc.merge_attention(c["out_ctx"], c["lse_ctx"], c["out_buf"], c["lse_buf"])
        torch.testing.assert_close(merged, c["merged"], atol=1e-6, rtol=1e-6)


def test_hybrid_attention_including_empty_buffer(ops):
    seen_empty = False
    for c in ops["attn"]:
        got = orc.hybrid_attention(c["q"], c["k_ctx"], c["v_ctx"], c["k_buf"], c["v_buf"])
        torch.testing.assert_close(got, c["hybrid"], atol=1e-6, rtol=1e-6)
        seen_empty |= c["k_buf"].shape[2] == 0
    assert seen_empty


def test_hybrid_equals_one_shot_softmax(ops):
    """Second witness: merged partials equal attention over concatenated K/V."""
    for c in ops["attn"]:
        B = c["q"].shape[0]
        k = torch.cat([c["k_ctx"].unsqueeze(0).expand(B, -1, -1, -1), c["k_buf"]], dim=2)
        v = torch.cat([c["v_ctx"].unsqueeze(0).expand(B, -1, -1, -1), c["v_buf"]], dim=2)
        full = orc.masked_attention(c["q"], k, v, None)
        torch.testing.assert_close(full, c["hybrid"], atol=1e-5, rtol=1e-5)


def test_teacher_forcing_mask_and_attention(ops):
    for c in ops["tf"]:
        Nt = c["num_targets"]
        mask = orc.teacher_forcing_buffer_mask(Nt)
        assert torch.equal(mask, c["mask"])
        out, lse = orc.buffer_attention(c["q"], c["k_buf"], c["v_buf"], mask=mask)
        torch.testing.assert_close(out, c["out_buf"], atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(lse, c["lse_buf"], atol=1e-6, rtol=1e-6)
        # first target row sees no buffer key: zero output, -inf lse
        assert torch.all(out[:, :, Nt] == 0) and torch.all(torch.isinf(lse[:, :, Nt]))
        got = orc.hybrid_teacher_forcing_attention(c["q"], c["k_ctx"], c["v_ctx"], c["k_buf"], c["v_buf"], Nt)
        torch.testing.assert_close(got, c["hybrid"], atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("name", ["config1.pt", "dh32.pt", "tiny_distinct.pt"])
def test_predictor_shared_backend(name):
    fx = load(name)
    p = orc.OraclePredictor(fx["state_dict"], fx["n_heads"])
    ys, ld, _ = p.sample_sequence(fx["xc"], fx["yc"], fx["xt"], fx["expo"], fx["normal"], shared=True)
    # identical draws for identical RNG streams
    torch.testing.assert_close(ys, fx["samples_shared"], atol=1e-5, rtol=1e-5)
    # the density AT a drawn value re-derives the normal variate from (y - mean) / std,
    # which amplifies fp32 rounding by 1/std: slightly looser than the 1e-5 of the joint density
    torch.testing.assert_close(ld, fx["sample_logdens_shared"], atol=3e-5, rtol=1e-5)
    for l, (k, v) in enumerate(fx["ctx_kv"]):
        torch.testing.assert_close(p.k_ctx[l][0], k, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(p.v_ctx[l][0], v, atol=1e-5, rtol=1e-5)
    jd = p.evaluate_joint_density(fx["xc"], fx["yc"], fx["xt"], fx["yt"], shared=True)
    torch.testing.assert_close(jd, fx["joint_logdens_shared"], atol=1e-5, rtol=0)


@pytest.mark.parametrize("name", ["config1.pt", "tiny_distinct.pt"])
def test_predictor_per_batch_context(name):
    """Per-batch context K/V = the reference's flex_attention backend."""
    fx = load(name)
    p = orc.OraclePredictor(fx["state_dict"], fx["n_heads"])
    ys, ld, _ = p.sample_sequence(fx["xc"], fx["yc"], fx["xt"], fx["expo"], fx["normal"], shared=False)
    torch.testing.assert_close(ys, fx["samples_flex"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(ld, fx["sample_logdens_flex"], atol=3e-5, rtol=1e-5)
    jd = p.evaluate_joint_density(fx["xc"], fx["yc"], fx["xt"], fx["yt"], shared=False)
    torch.testing.assert_close(jd, fx["joint_logdens_flex"], atol=1e-5, rtol=0)


def test_variate_order_reproduces_global_generator():
    """draw_variates replays what torch.multinomial + randn_like consume."""
    B, K, Nt = 5, 4, 3
    w = torch.softmax(torch.randn(B, K, generator=torch.Generator().manual_seed(1)), -1)
    torch.manual_seed(123)
    want = []
    for _ in range(Nt):
        idx = torch.multinomial(w, 1, replacement=True)
        want.append((idx, torch.randn(B, 1, 1, 1)))
    expo, normal = orc.draw_variates(123, Nt, B, K)
    for t in range(Nt):
        assert torch.equal((w / expo[t]).argmax(-1, keepdim=True), want[t][0])
        assert torch.equal(normal[t], want[t][1].view(B))


def test_forward_masked_matches_reference_forward():
    """The oracle's masked forward against the reference's training forward
    (ARTabPFN.forward under create_row_mask, and under the inference-style mask
    of the reference's own test) run on CPU: per-target log density and loss."""
    for c in load("forward.pt"):
        o = orc.OraclePredictor(c["state_dict"], c["n_heads"])
        if c["attending_chunks"] != "tf":
            assert orc.row_mask_visible(c["xb"].shape[1], c["xt"].shape[1], c["attending_chunks"]) == c["visible"]
        ld = o.forward_masked(c["xc"], c["yc"], c["xb"], c["yb"], c["xt"], c["yt"], c["visible"], shared=False)
        sd64 = {k: v.double() for k, v in c["state_dict"].items()}
        d = lambda k: c[k].double()
        ld64 = orc.OraclePredictor(sd64, c["n_heads"]).forward_masked(d("xc"), d("yc"), d("xb"), d("yb"), d("xt"),
                                                                      d("yt"), c["visible"], shared=False)
        noise = (c["logdens"].double() - ld64).abs().float()     # the reference's own fp32 rounding
        assert ((ld - c["logdens"]).abs() <= 1e-5 + 2 * noise).all(), (c["name"], (ld - c["logdens"]).abs().max())
        torch.testing.assert_close(-ld.mean(), c["loss"], atol=1e-5, rtol=1e-5)


def test_forward_tf_style_equals_joint_density():
    """With buffer = target data and the inference-style mask the forward is the teacher-forced
    joint density (the reference's test_teacher_forcing_matches_forward)."""
    c = [x for x in load("forward.pt") if x["name"] == "tf_style"][0]
    o = orc.OraclePredictor(c["state_dict"], c["n_heads"])
    a = o.forward_masked(c["xc"], c["yc"], c["xt"], c["yt"], c["xt"], c["yt"], c["visible"], shared=False)
    b = o.evaluate_joint_density(c["xc"], c["yc"], c["xt"], c["yt"], shared=False)
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)


def test_row_mask_factory_matches_oracle():
    """The shipped create_row_mask (host logic, no GPU) lists the same counts as the oracle."""
    from ar_tabpfn.model import create_row_mask
    from ar_tabpfn.model.attention import RowMask
    for Nc, Nb, Nt, ch in [(10, 4, 16, None), (50, 8, 32, 3), (33, 3, 12, None), (5, 0, 4, None), (7, 2, 5, 1)]:
        m = create_row_mask(num_rows=Nc + Nb + Nt, context_len=Nc, buffer_len=Nb, attending_chunks=ch, device="cpu")
        assert m.visible == orc.row_mask_visible(Nb, Nt, ch)
    assert RowMask.teacher_forcing(8, 4).visible == [1, 2, 3, 4, 0, 1, 2, 3]
    with pytest.raises(ValueError):
        create_row_mask(num_rows=5, context_len=4, buffer_len=3)


def test_ragged_buffer_attention_matches_reference():
    """Masked buffer attention and hybrid attention with one visible prefix per stream
    (lengths 0 .. Nb), against the reference's eager operators."""
    for c in load("ragged.pt"):
        out, lse = orc.buffer_attention(c["q"], c["k_buf"], c["v_buf"], mask=c["mask"])
        torch.testing.assert_close(out, c["out_buf"], atol=1e-6, rtol=1e-6)
        assert torch.equal(torch.isinf(lse), torch.isinf(c["lse_buf"]))
        fin = torch.isfinite(lse)
        torch.testing.assert_close(lse[fin], c["lse_buf"][fin], atol=1e-6, rtol=1e-6)
        assert (out[c["lens"] == 0] == 0).all()          # nothing visible: zero output
        hyb = orc.hybrid_attention(c["q"], c["k_ctx"], c["v_ctx"], c["k_buf"], c["v_buf"], buf_mask=c["mask"])
        torch.testing.assert_close(hyb, c["hybrid"], atol=1e-6, rtol=1e-6)


def test_backbone_with_column_tokens_matches_reference():
    """C > 1 column tokens per row: the oracle's backbone against golden outputs of the reference's
    TwoStageTransformer under create_dense_mask / create_row_mask."""
    for c in load("columns.pt"):
        vis = orc.row_mask_visible(c["Nb"], c["Nt"], c["attending_chunks"])
        out, kvs = orc.backbone_forward(c["state_dict"], c["cfg"]["n_heads"], c["x"], c["Nc"], c["Nb"], vis)
        torch.testing.assert_close(out, c["out"], atol=5e-6, rtol=1e-5)
        torch.testing.assert_close(kvs[0][0], c["k0"], atol=2e-6, rtol=1e-5)
        torch.testing.assert_close(kvs[0][1], c["v0"], atol=2e-6, rtol=1e-5)
