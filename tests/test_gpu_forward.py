"""GPU parity of the masked forward (ARTabPFN.forward for inference -> predictor ->
artab_forward_masked) against golden outputs of the reference's training forward and
against the CPU oracle."""
import pytest
import torch

import artab_oracle as orc
from util import build_model, load_golden

pytestmark = pytest.mark.gpu


def _call(m, c, mask, dev=lambda t: t.cuda()):
    from ar_tabpfn.model import create_dense_mask
    return m(x_context=dev(c["xc"]), y_context=dev(c["yc"]), x_buffer=dev(c["xb"]), y_buffer=dev(c["yb"]),
             x_target=dev(c["xt"]), mask_features=create_dense_mask(seq_len=1, device="cuda"), mask_rows=mask,
             y_target=dev(c["yt"]))


def _mask(c):
    from ar_tabpfn.model import create_row_mask
    from ar_tabpfn.model.attention import RowMask
    Nc, Nb, Nt = c["xc"].shape[1], c["xb"].shape[1], c["xt"].shape[1]
    if c["attending_chunks"] == "tf":
        return RowMask.teacher_forcing(Nc, Nt)
    return create_row_mask(num_rows=Nc + Nb + Nt, context_len=Nc, buffer_len=Nb,
                           attending_chunks=c["attending_chunks"], device="cuda")


def test_forward_fp32_matches_reference_golden():
    """fp32: per-target log density within 1e-5 of the reference's forward (widened only by the
    reference's own distance from an fp64 evaluation), loss within 1e-5."""
    for c in load_golden("forward.pt"):
        m, _ = build_model(c)
        loss = _call(m, c, _mask(c))
        ld = m.last_logdens.cpu()
        sd64 = {k: v.double() for k, v in c["state_dict"].items()}
        d = lambda k: c[k].double()
        ld64 = orc.OraclePredictor(sd64, c["n_heads"]).forward_masked(d("xc"), d("yc"), d("xb"), d("yb"), d("xt"),
                                                                      d("yt"), c["visible"], shared=False)
        noise = (c["logdens"].double() - ld64).abs().float()
        assert ((ld - c["logdens"]).abs() <= 1e-5 + 2 * noise).all(), (c["name"], (ld - c["logdens"]).abs().max())
        torch.testing.assert_close(loss.cpu(), c["loss"], atol=1e-5, rtol=1e-5)
        # a second call on the same model reuses the predictor and its caches
        loss2 = _call(m, c, _mask(c))
        assert torch.equal(loss2, loss)


def test_forward_bf16_within_tolerance():
    """bf16 caches and tensor-core kernels (head_dim 32) against the fp32 oracle on
    bf16-representable weights and inputs: per-target log density within 2e-3.  Data: the
    head_dim 32 fixture, its last context rows taken as buffer rows."""
    from ar_tabpfn.model import ARTabPFNPredictor
    fx = load_golden("dh32.pt")
    m, sd = build_model(fx, bf16_round=True)
    r = {k: fx[k].to(torch.bfloat16).float() for k in ("xc", "yc", "xt", "yt")}
    Nt = r["xt"].shape[1]
    for Nb, chunks in [(4, 2), (6, None)]:
        xc, yc, xb, yb = r["xc"][:, :-Nb], r["yc"][:, :-Nb], r["xc"][:, -Nb:], r["yc"][:, -Nb:]
        vis = orc.row_mask_visible(Nb, Nt, chunks)
        for backend, shared in (("flex_attention", False), ("triton_shared_context", True)):
            want = orc.OraclePredictor(sd, fx["n_heads"]).forward_masked(xc, yc, xb, yb, r["xt"], r["yt"], vis,
                                                                         shared=shared)
            p = ARTabPFNPredictor.from_trained_model(m, backend=backend, precision="bf16")
            ld = p.forward_masked(xc.cuda(), yc.cuda(), xb.cuda(), yb.cuda(), r["xt"].cuda(), r["yt"].cuda(), vis)
            assert (ld.cpu() - want).abs().max() <= 2e-3, (Nb, backend, (ld.cpu() - want).abs().max())


def test_forward_bf16_sensitive_case_no_worse_than_rounding():
    """A case where bf16 storage of q, k, v alone (emulated on the CPU oracle, everything else
    fp32) already moves the log density by more than 2e-3 (50 context rows, one dataset per
    element): the device result must not be further from the fp32 oracle than that emulation."""
    from ar_tabpfn.model import ARTabPFNPredictor
    c = [x for x in load_golden("forward.pt") if x["name"] == "dh32_three_chunks"][0]
    m, sd = build_model(c, bf16_round=True)
    r = {k: c[k].to(torch.bfloat16).float() for k in ("xc", "yc", "xb", "yb", "xt", "yt")}
    args = (r["xc"], r["yc"], r["xb"], r["yb"], r["xt"], r["yt"], c["visible"])
    want = orc.OraclePredictor(sd, c["n_heads"]).forward_masked(*args, shared=False)
    emu = orc.OraclePredictor(sd, c["n_heads"], orc.Emulation(qkv=True)).forward_masked(*args, shared=False)
    floor = (emu - want).abs().max()
    assert floor > 2e-3
    p = ARTabPFNPredictor.from_trained_model(m, backend="flex_attention", precision="bf16")
    ld = p.forward_masked(*[a.cuda() for a in args[:6]], c["visible"]).cpu()
    assert (ld - want).abs().max() <= floor, ((ld - want).abs().max(), floor)
    assert (ld - want).abs().mean() <= 2e-3


def test_forward_tf_mask_equals_joint_density():
    """Buffer = target data under the inference-style mask gives the teacher-forced density
    (the reference's test_teacher_forcing_matches_forward), here through two different kernels
    paths of the buffer pass."""
    from ar_tabpfn.model import ARTabPFNPredictor
    c = [x for x in load_golden("forward.pt") if x["name"] == "tf_style"][0]
    m, _ = build_model(c)
    p = ARTabPFNPredictor.from_trained_model(m)
    g = {k: c[k].cuda() for k in ("xc", "yc", "xt", "yt")}
    a = p.forward_masked(g["xc"], g["yc"], g["xt"], g["yt"], g["xt"], g["yt"], c["visible"])
    b = p.evaluate_joint_density(g["xc"], g["yc"], g["xt"], g["yt"])
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)


def test_forward_argument_errors():
    from ar_tabpfn.model import create_row_mask
    c = load_golden("forward.pt")[0]
    m, _ = build_model(c)
    Nc, Nb, Nt = c["xc"].shape[1], c["xb"].shape[1], c["xt"].shape[1]
    with pytest.raises(ValueError):      # mask built for other row counts
        _call(m, c, create_row_mask(num_rows=Nc + Nb + Nt + 1, context_len=Nc, buffer_len=Nb))
    with pytest.raises(TypeError):       # not a RowMask
        _call(m, c, object())
    # more buffer rows than AR position tokens: the reference's broadcast fails too
    big = dict(c)
    big["xb"] = torch.randn(c["xb"].shape[0], 5, c["xb"].shape[2])
    big["yb"] = torch.randn(c["xb"].shape[0], 5)
    with pytest.raises(ValueError):
        _call(m, big, create_row_mask(num_rows=Nc + 5 + Nt, context_len=Nc, buffer_len=5))
    # no y_target: no loss, like the reference
    from ar_tabpfn.model import create_dense_mask
    assert m(c["xc"].cuda(), c["yc"].cuda(), c["xb"].cuda(), c["yb"].cuda(), c["xt"].cuda(),
             create_dense_mask(1), _mask(c)) is None


def test_forward_without_buffer_rows():
    """Nb = 0: every target sees the context only (no private cache is laid out at all)."""
    from ar_tabpfn.model import ARTabPFNPredictor
    c = load_golden("forward.pt")[2]
    m, sd = build_model(c)
    B, F = c["xt"].shape[0], c["xt"].shape[2]
    xb, yb = torch.zeros(B, 0, F), torch.zeros(B, 0)
    vis = [0] * c["xt"].shape[1]
    for backend, shared in (("flex_attention", False), ("triton_shared_context", True)):
        want = orc.OraclePredictor(sd, c["n_heads"]).forward_masked(c["xc"], c["yc"], xb, yb, c["xt"], c["yt"], vis,
                                                                     shared=shared)
        p = ARTabPFNPredictor.from_trained_model(m, backend=backend)
        got = p.forward_masked(c["xc"].cuda(), c["yc"].cuda(), xb.cuda(), yb.cuda(), c["xt"].cuda(), c["yt"].cuda(),
                               vis)
        torch.testing.assert_close(got.cpu(), want, atol=2e-5, rtol=1e-5)
