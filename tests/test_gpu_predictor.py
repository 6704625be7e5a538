"""GPU parity of the whole path (predictor API -> C ABI -> kernels) against the
golden outputs of the reference and against the CPU oracle."""
import pytest
import torch

import artab_oracle as orc
from util import build_model, load_golden

pytestmark = pytest.mark.gpu

BF16_LOGDENS_ATOL = 2e-3


def fp64_joint_density(fx, shared):
    sd = {k: v.double() for k, v in fx["state_dict"].items()}
    d = lambda k: fx[k].double()
    return orc.OraclePredictor(sd, fx["n_heads"]).evaluate_joint_density(d("xc"), d("yc"), d("xt"), d("yt"),
                                                                         shared=shared)


def predictor(m, backend, precision=None):
    from ar_tabpfn.model import ARTabPFNPredictor
    return ARTabPFNPredictor.from_trained_model(m, backend=backend, precision=precision)


@pytest.mark.parametrize("name", ["config1.pt", "dh32.pt", "tiny_distinct.pt"])
@pytest.mark.parametrize("backend,tag", [("triton_shared_context", "shared"), ("flex_attention", "flex")])
def test_fp32_matches_reference_golden(name, backend, tag):
    """fp32 mode: identical draws for identical RNG streams, log density within 1e-5."""
    fx = load_golden(name)
    m, _ = build_model(fx)
    p = predictor(m, backend)
    c = lambda k: fx[k].cuda()
    ys = p.sample_sequence(c("xc"), c("yc"), c("xt"), variates=(c("expo"), c("normal")))
    torch.testing.assert_close(ys.cpu(), fx[f"samples_{tag}"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(p.last_logdens.cpu(), fx[f"sample_logdens_{tag}"], atol=3e-5, rtol=1e-5)
    if tag == "shared":
        for l, (k, v) in enumerate(fx["ctx_kv"]):
            layer = m.backbone.layers[l]
            torch.testing.assert_close(layer.k_ctx_cache.cpu(), k, atol=1e-5, rtol=1e-5)
            torch.testing.assert_close(layer.v_ctx_cache.cpu(), v, atol=1e-5, rtol=1e-5)
        assert p.buffer_len == fx["xt"].shape[1] - 1 and p.context_len == fx["xc"].shape[1]
    jd = p.evaluate_joint_density(c("xc"), c("yc"), c("xt"), c("yt")).cpu()
    # 1e-5 absolute, widened only where the reference's own fp32 result sits further than that
    # from an fp64 evaluation of the same algorithm (ill-conditioned targets: sharp mixtures)
    want = fx[f"joint_logdens_{tag}"]
    noise = (want.double() - fp64_joint_density(fx, tag == "shared")).abs().float()
    assert ((jd - want).abs() <= 1e-5 + 2 * noise).all(), (jd - want).abs().max()
    assert ((jd - want).abs() <= 1e-5).float().mean() > 0.9


def test_bf16_mode_within_tolerance():
    """bf16 mode against the fp32 oracle on bf16-representable weights and inputs:
    per-target log density within 2e-3 absolute."""
    fx = load_golden("dh32.pt")
    m, sd = build_model(fx, bf16_round=True)
    r = lambda k: fx[k].to(torch.bfloat16).float()
    xc, yc, xt, yt = r("xc"), r("yc"), r("xt"), r("yt")
    want = orc.OraclePredictor(sd, fx["n_heads"]).evaluate_joint_density(xc, yc, xt, yt)
    for backend in ("triton_shared_context", "flex_attention"):
        p = predictor(m, backend, precision="bf16")
        got = p.evaluate_joint_density(xc.cuda(), yc.cuda(), xt.cuda(), yt.cuda())
        torch.testing.assert_close(got.cpu(), want, atol=BF16_LOGDENS_ATOL, rtol=0)
    p = predictor(m, "triton_shared_context", precision="bf16")
    ys = p.sample_sequence(xc.cuda(), yc.cuda(), xt.cuda(), variates=(fx["expo"].cuda(), fx["normal"].cuda()))
    wy, wl, wc = orc.OraclePredictor(sd, fx["n_heads"]).sample_sequence(xc, yc, xt, fx["expo"], fx["normal"])
    same = p.last_components.cpu() == wc
    assert same.float().mean() > 0.95
    first_flip = (~same).float().argmax(dim=1)
    for b in range(ys.shape[0]):  # compare each stream up to its first differing component choice
        n = int(first_flip[b]) if (~same[b]).any() else ys.shape[1]
        torch.testing.assert_close(ys[b, :n].cpu(), wy[b, :n], atol=5e-3, rtol=5e-3)


def test_step_api_matches_oracle():
    """transformer_decode / autoregressive_decode (the reference's step-level API)."""
    fx = load_golden("config1.pt")
    m, sd = build_model(fx)
    p = predictor(m, "triton_shared_context")
    o = orc.OraclePredictor(sd, fx["n_heads"])
    xc, yc, xt, yt = fx["xc"], fx["yc"], fx["xt"], fx["yt"]
    B, Nt, _ = xt.shape
    p.init_kv_cache(B, Nt, torch.device("cuda"), torch.float32)
    p.prefill_context(xc.cuda(), yc.cuda())
    o.prefill(xc, yc, shared=True)
    for t in range(4):
        tgt = orc.embed_rows(sd, xt[:, t:t + 1], None, orc.MARKER_TARGET)
        if t == 0:
            emb, commit = tgt, 0
        else:
            ar = torch.full((B, 1), t % o.S, dtype=torch.long)
            emb = torch.cat([orc.embed_rows(sd, xt[:, t - 1:t], yt[:, t - 1:t], orc.MARKER_BUFFER, ar), tgt], 1)
            commit = 1
        z = p.transformer_decode(emb.cuda(), commit)
        torch.testing.assert_close(z.cpu(), o.decode(emb, commit), atol=2e-5, rtol=1e-5)
        assert p.buffer_len == o.buffer_len and p.seq_len == xc.shape[1] + o.buffer_len
    with pytest.raises(ValueError):
        p.transformer_decode(torch.zeros(B, 3, 64, device="cuda"), 0)
    torch.manual_seed(0)
    y = p.autoregressive_decode(xt[:, 4:5].cuda(), xt[:, 3:4].cuda(), yt[:, 3:4].cuda(), ar_idx=4)
    assert y.shape == (B, 1) and torch.isfinite(y).all()


def test_errors_like_reference():
    fx = load_golden("tiny_distinct.pt")
    m, _ = build_model(fx)
    with pytest.raises(ValueError, match="Unsupported backend"):
        predictor(m, "triton")
    p = predictor(m, "triton_shared_context")
    B, Nt = fx["xt"].shape[:2]
    p.init_kv_cache(B, 1, torch.device("cuda"), torch.float32)
    p.prefill_context(fx["xc"].cuda(), fx["yc"].cuda())
    emb = torch.zeros(B, 2, 32, device="cuda")
    p.transformer_decode(emb, 1)
    with pytest.raises(ValueError, match="buffer cache exceeded"):
        p.transformer_decode(emb, 1)


def test_deterministic_and_stream_independent():
    """Run-to-run bitwise determinism, and a stream's result does not depend on which
    other streams share the batch (size-independent property used at full sizes)."""
    fx = load_golden("dh32.pt")
    m, _ = build_model(fx)
    c = lambda k: fx[k].cuda()
    for prec in ("fp32", "bf16"):
        p = predictor(m, "triton_shared_context", precision=prec)
        a = p.sample_sequence(c("xc"), c("yc"), c("xt"), variates=(c("expo"), c("normal"))).clone()
        la = p.last_logdens.clone()
        b = p.sample_sequence(c("xc"), c("yc"), c("xt"), variates=(c("expo"), c("normal")))
        assert torch.equal(a, b) and torch.equal(la, p.last_logdens)
        sub = p.sample_sequence(c("xc")[2:5], c("yc")[2:5], c("xt")[2:5],
                                variates=(c("expo")[:, 2:5], c("normal")[:, 2:5]))
        torch.testing.assert_close(sub, a[2:5], atol=1e-5, rtol=1e-5)


def test_dependent_launch_is_bit_identical_to_serialised_launch():
    """The overlapped launch mode (kernels begin while their predecessor drains, the buffer
    pass runs beside the context contraction) must not change a single bit."""
    from ar_tabpfn import _lib
    lib = _lib.lib()
    fx = load_golden("dh32.pt")
    m, _ = build_model(fx)
    c = lambda k: fx[k].cuda()
    try:
        for prec in ("fp32", "bf16"):
            p = predictor(m, "triton_shared_context", precision=prec)
            got = {}
            for on in (1, 0, 1):
                lib.artab_set_dependent_launch(on)
                ys = p.sample_sequence(c("xc"), c("yc"), c("xt"), variates=(c("expo"), c("normal"))).clone()
                jd = p.evaluate_joint_density(c("xc"), c("yc"), c("xt"), c("yt")).clone()
                torch.cuda.synchronize()
                if not got:
                    got = {"ys": ys, "ld": p.last_logdens.clone(), "jd": jd}
                else:
                    assert torch.equal(ys, got["ys"]) and torch.equal(jd, got["jd"])
    finally:
        lib.artab_set_dependent_launch(1)


def test_sampler_density_equals_teacher_forcing_with_shifted_ar_index():
    """Round trip: the density the sampler assigned to its own draws equals the
    teacher-forced density of those draws when the AR-token index convention is
    aligned (the sampler adds ar_tokens[t mod S] to the buffer carrying datum t-1,
    teacher forcing adds ar_tokens[j mod S] to the buffer carrying datum j)."""
    fx = load_golden("config1.pt")
    m, _ = build_model(fx)
    with torch.no_grad():
        m.ar_tokens.zero_()          # removes the index shift between the two paths
    p = predictor(m, "triton_shared_context")
    c = lambda k: fx[k].cuda()
    ys = p.sample_sequence(c("xc"), c("yc"), c("xt"), variates=(c("expo"), c("normal")))
    ld = p.last_logdens.clone()
    jd = p.evaluate_joint_density(c("xc"), c("yc"), c("xt"), ys)
    torch.testing.assert_close(jd, ld, atol=5e-5, rtol=1e-5)
