"""The benchmarked configurations at their full sizes (bf16 mode): the device against the CPU
oracle on a subset of streams / datasets that the oracle finishes in seconds (streams are
independent given the context, so a subset is checked exactly as the whole would be), plus
size-independent properties of the whole job.  Models and rows come from synthetic.py, the
module the benchmark itself builds its workload from."""
import pytest
import torch

import artab_oracle as orc
import synthetic as syn

pytestmark = pytest.mark.gpu

BF16_LOGDENS_ATOL = 2e-3   # per target, absolute: the bar of the bf16 mode, no target excused


def _sd(m):
    return {k: v.detach().cpu().clone() for k, v in m.state_dict().items()}


def _predictor(m, backend):
    from ar_tabpfn.model import ARTabPFNPredictor
    return ARTabPFNPredictor.from_trained_model(m, backend=backend, precision="bf16")


def test_config3_benchmark_job_against_oracle():
    """The exact job bench.py times (same model, rows, stream count and random numbers): teacher-forced
    log density of all 512 streams and the sampled trajectories of streams 0, 1, 300 and 511 against
    the fp32 oracle on the same bf16-representable weights and inputs."""
    c = syn.CONFIG3
    B, Nt, H = c["streams"], c["n_targets"], syn.MODEL_6L["n_heads"]
    m = syn.config3_model()
    sd = _sd(m)
    p = _predictor(m.cuda(), "triton_shared_context")
    xc, yc, xt = syn.config3_workload(B)
    yt = syn.config3_rows()[3].expand(B, -1).contiguous()
    dev = torch.device("cuda")
    expo, normal = syn.variates(c["seed"], Nt, B, syn.MODEL_6L["num_components"], dev)
    ys = p.sample_sequence(xc.to(dev), yc.to(dev), xt.to(dev), variates=(expo, normal)).clone()
    ld, comp = p.last_logdens.clone(), p.last_components.clone()
    assert int(p._bufs["status"].item()) == 0
    # (1) teacher forcing on the dataset's own labels: every stream holds the same rows, so one
    # oracle stream is the reference of all 512
    jd = p.evaluate_joint_density(xc.to(dev), yc.to(dev), xt.to(dev), yt.to(dev)).cpu()
    want = orc.OraclePredictor(sd, H).evaluate_joint_density(xc[:1], yc[:1], xt[:1], yt[:1])
    err = (jd - want).abs()
    print("config 3 teacher forcing: max |d| %.2e, median %.2e over %d targets" % (err.max(), err.median(), err.numel()))
    assert float(err.max()) <= BF16_LOGDENS_ATOL
    # (2) sampling: identical draws for identical random numbers.  The chosen mixture components
    # must agree for the whole trajectory (a flip would fork it); values and the sampler's own log
    # density then agree to rounding.
    pick = [0, 1, 300, 511]
    wy, wl, wc = orc.OraclePredictor(sd, H).sample_sequence(xc[pick], yc[pick], xt[pick], expo[:, pick].cpu(),
                                                            normal[:, pick].cpu())
    assert torch.equal(comp[pick].cpu(), wc)
    dy, dl = (ys[pick].cpu() - wy).abs(), (ld[pick].cpu() - wl).abs()
    print("config 3 sampling, 4 streams x %d steps: max |dy| %.2e, max |d logdens| %.2e" % (Nt, dy.max(), dl.max()))
    assert float(dy.max()) <= 1e-3 and float(dl.max()) <= BF16_LOGDENS_ATOL
    # (3) teacher forcing on the device's own samples (different rows per stream), same four streams
    jd2 = p.evaluate_joint_density(xc.to(dev), yc.to(dev), xt.to(dev), ys).cpu()
    want2 = orc.OraclePredictor(sd, H).evaluate_joint_density(xc[pick], yc[pick], xt[pick], ys[pick].cpu())
    e2 = (jd2[pick] - want2).abs()
    print("config 3 teacher forcing on sampled rows: max |d| %.2e" % e2.max())
    assert float(e2.max()) <= BF16_LOGDENS_ATOL


def test_config4_two_datasets_against_oracle():
    """Config 4 at full size (64 independent datasets x (2048 context rows + 256 targets), one
    context per dataset) on the device; datasets 0 and 41 against the oracle's per-dataset
    ("flex_attention") semantics."""
    H = syn.MODEL_6L["n_heads"]
    m = syn.config4_model()
    sd = _sd(m)
    p = _predictor(m.cuda(), "flex_attention")
    xc, yc, xt, yt = syn.config4_workload()
    jd = p.evaluate_joint_density(xc.cuda(), yc.cuda(), xt.cuda(), yt.cuda()).cpu()
    assert int(p._bufs["status"].item()) == 0
    pick = [0, 41]
    want = orc.OraclePredictor(sd, H).evaluate_joint_density(xc[pick], yc[pick], xt[pick], yt[pick], shared=False)
    err = (jd[pick] - want).abs()
    print("config 4, 2 of 64 datasets: max |d| %.2e, median %.2e over %d targets" % (err.max(), err.median(), err.numel()))
    assert float(err.max()) <= BF16_LOGDENS_ATOL
    # the per-dataset sums the configuration reports
    assert float((jd[pick].sum(1) - want.sum(1)).abs().max()) <= 2e-2


def test_config5_full_context_against_oracle():
    """Config 5's context at full size (16384 rows x 100 features) with two streams x eight targets:
    teacher forcing and sampling against the oracle (its prefill walks the query rows in chunks)."""
    H, K = syn.MODEL_6L["n_heads"], syn.MODEL_6L["num_components"]
    m = syn.config5_model()
    sd = _sd(m)
    p = _predictor(m.cuda(), "triton_shared_context")
    xcr, ycr, xtr, ytr = syn.config5_rows(n_targets=8)
    B, Nt = 2, 8
    xc, yc = xcr.expand(B, -1, -1), ycr.expand(B, -1)
    xt, yt = xtr.expand(B, -1, -1).contiguous(), ytr.expand(B, -1).contiguous()
    dev = torch.device("cuda")
    jd = p.evaluate_joint_density(xc.to(dev), yc.to(dev), xt.to(dev), yt.to(dev)).cpu()
    expo, normal = syn.variates(syn.CONFIG5["seed"], Nt, B, K, dev)
    ys = p.sample_sequence(xc.to(dev), yc.to(dev), xt.to(dev), variates=(expo, normal)).cpu()
    ld, comp = p.last_logdens.cpu(), p.last_components.cpu()
    assert int(p._bufs["status"].item()) == 0
    o = orc.OraclePredictor(sd, H)
    want = o.evaluate_joint_density(xc[:1], yc[:1], xt[:1], yt[:1])
    err = (jd - want).abs()
    print("config 5 teacher forcing (16384-row context): max |d| %.2e" % err.max())
    assert float(err.max()) <= BF16_LOGDENS_ATOL
    wy, wl, wc = orc.OraclePredictor(sd, H).sample_sequence(xc, yc, xt, expo.cpu(), normal.cpu())
    assert torch.equal(comp, wc)
    print("config 5 sampling: max |dy| %.2e, max |d logdens| %.2e" % ((ys - wy).abs().max(), (ld - wl).abs().max()))
    assert float((ys - wy).abs().max()) <= 1e-3 and float((ld - wl).abs().max()) <= BF16_LOGDENS_ATOL


def _setup():
    c = syn.CONFIG3
    m = syn.config3_model().cuda()
    with torch.no_grad():
        m.ar_tokens.zero_()   # aligns the AR-index convention of sampling and teacher forcing
    p = _predictor(m, "triton_shared_context")
    xc, yc, xt = (t.cuda() for t in syn.config3_workload(c["streams"]))
    expo, normal = syn.variates(c["seed"], c["n_targets"], c["streams"], syn.MODEL_6L["num_components"], "cuda")
    expo[:, 1], normal[:, 1] = expo[:, 0], normal[:, 0]          # streams 0 and 1: same random numbers
    expo[:, 300], normal[:, 300] = expo[:, 0], normal[:, 0]      # ... and one in another row tile
    return p, xc, yc, xt, (expo, normal)


def test_config3_full_size_round_trips():
    p, xc, yc, xt, var = _setup()
    ys = p.sample_sequence(xc, yc, xt, variates=var).clone()
    ld = p.last_logdens.clone()
    assert int(p._bufs["status"].item()) == 0
    assert torch.isfinite(ys).all() and torch.isfinite(ld).all()
    # same context, same inputs, same random numbers => same trajectory, wherever the stream sits
    assert torch.equal(ys[0], ys[1]) and torch.equal(ld[0], ld[1])
    assert torch.equal(ys[0], ys[300]) and torch.equal(ld[0], ld[300])
    # streams with different random numbers differ
    assert not torch.equal(ys[0], ys[2])
    # run-to-run bitwise determinism
    ys2 = p.sample_sequence(xc, yc, xt, variates=var)
    assert torch.equal(ys, ys2) and torch.equal(ld, p.last_logdens)
    # a stream's result does not depend on the batch it rides in (other tile shapes and split
    # plans regroup fp32 sums, so compare with the bf16-mode tolerance; a flipped mixture
    # component would show as an O(1) difference)
    sub = p.sample_sequence(xc[:96], yc[:96], xt[:96], variates=(var[0][:, :96].contiguous(),
                                                                  var[1][:, :96].contiguous()))
    close = ((sub - ys[:96]).abs() <= 2e-3).all(dim=1)
    assert close.float().mean() >= 0.97, float(close.float().mean())
    # sampler density == teacher-forced density of its own draws (two different kernels paths:
    # 128 incremental steps with in-place KV append vs one block-causal pass)
    jd = p.evaluate_joint_density(xc, yc, xt, ys)
    err = (jd - ld).abs()
    assert float(err.median()) < 1e-3
    assert float((err <= 4e-3).float().mean()) >= 0.999, float(err.max())
    assert int(p._bufs["status"].item()) == 0


def test_config4_full_size_properties():
    """Teacher-forced joint density at the fourth configuration's full size: 64 independent
    datasets x (2048 context rows + 256 targets) x 20 features, the 6-layer d_model 192 model,
    one context per dataset.  Properties: finite, bitwise repeatable, each dataset's result
    independent of the batch it rides in, and the bf16 mode within its tolerance of the fp32 mode."""
    import ar_tabpfn
    dev = torch.device("cuda")
    model = syn.config4_model().to(dev)
    B, Nc, Nt = syn.CONFIG4["datasets"], syn.CONFIG4["n_ctx"], syn.CONFIG4["n_targets"]
    xc, yc, xt, yt = (t.to(dev) for t in syn.config4_workload())
    p16 = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="flex_attention", precision="bf16")
    ld = p16.evaluate_joint_density(xc, yc, xt, yt).clone()
    assert ld.shape == (B, Nt) and torch.isfinite(ld).all() and int(p16._bufs["status"].item()) == 0
    assert torch.equal(ld, p16.evaluate_joint_density(xc, yc, xt, yt))
    sub = p16.evaluate_joint_density(xc[5:13], yc[5:13], xt[5:13], yt[5:13])
    err = (sub - ld[5:13]).abs()
    assert float(err.median()) <= 1e-3 and float((err <= 4e-3).float().mean()) >= 0.99, float(err.max())
    # every dataset reads its own context: new labels in one context move that dataset's result only
    yc2 = yc.clone()
    yc2[7] = yc2[7] * -2.0 + 3.0
    ch = p16.evaluate_joint_density(xc, yc2, xt, yt)
    keep = [b for b in range(B) if b != 7]
    assert torch.equal(ch[keep], ld[keep])
    assert float((ch[7] - ld[7]).abs().max()) > 1e-2
    p32 = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="flex_attention", precision="fp32")
    ld32 = p32.evaluate_joint_density(xc, yc, xt, yt)
    err = (ld - ld32).abs()
    assert float(err.median()) <= 1e-3 and float((err <= 2e-3).float().mean()) >= 0.95, (float(err.max()),
                                                                                          float(err.median()))
    # the per-dataset sums the configuration reports
    assert float((ld.sum(1) - ld32.sum(1)).abs().max()) <= 2e-3 * Nt


def test_config5_full_context_properties():
    """The fifth configuration's context at full size (16384 rows x 100 features, 20 % product
    columns, shared by all streams) with a reduced job (256 streams x 12 targets): finite, bitwise
    repeatable, streams with equal random numbers equal wherever they sit, sampler density equal
    to the teacher-forced density of its own draws."""
    import ar_tabpfn
    dev = torch.device("cuda")
    model = syn.config5_model().to(dev)
    with torch.no_grad():
        model.ar_tokens.zero_()
    p = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="triton_shared_context", precision="bf16")
    B, Nc, Nt = 256, 16384, 12
    xcr, ycr, xtr, _ = syn.config5_rows(n_targets=Nt)
    xc, yc = xcr.to(dev).expand(B, -1, -1), ycr.to(dev).expand(B, -1)
    xt = xtr.to(dev).expand(B, -1, -1).contiguous()
    gd = torch.Generator(device=dev).manual_seed(4)
    expo = torch.empty(Nt, B, 5, device=dev).exponential_(1.0, generator=gd)
    normal = torch.randn(Nt, B, device=dev, generator=gd)
    expo[:, 1], normal[:, 1] = expo[:, 0], normal[:, 0]
    expo[:, 200], normal[:, 200] = expo[:, 0], normal[:, 0]
    ys = p.sample_sequence(xc, yc, xt, variates=(expo, normal)).clone()
    ld = p.last_logdens.clone()
    assert torch.isfinite(ys).all() and torch.isfinite(ld).all() and int(p._bufs["status"].item()) == 0
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[200]) and not torch.equal(ys[0], ys[2])
    assert torch.equal(ys, p.sample_sequence(xc, yc, xt, variates=(expo, normal)))
    jd = p.evaluate_joint_density(xc, yc, xt, ys)
    err = (jd - ld).abs()
    assert float(err.median()) < 1e-3 and float((err <= 4e-3).float().mean()) >= 0.99, float(err.max())
