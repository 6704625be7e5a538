"""Size-independent properties of the path at the benchmark's full size (config 3:
512 sample streams x 128 targets over a 1024-row shared context, bf16 mode), where the
CPU oracle would need minutes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup():
    import bench
    from ar_tabpfn.model import ARTabPFNPredictor
    m = bench.build_model().cuda()
    with torch.no_grad():
        m.ar_tokens.zero_()   # aligns the AR-index convention of sampling and teacher forcing
    p = ARTabPFNPredictor.from_trained_model(m, backend="triton_shared_context", precision="bf16")
    xc, yc, xt = (t.cuda() for t in bench.workload(bench.STREAMS))
    g = torch.Generator(device="cuda").manual_seed(bench.SEED)
    K = bench.CFG["num_components"]
    expo = torch.empty(bench.NT, bench.STREAMS, K, device="cuda").exponential_(1.0, generator=g)
    normal = torch.randn(bench.NT, bench.STREAMS, device="cuda", generator=g)
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
    import microbench as mb
    import ar_tabpfn
    dev = torch.device("cuda")
    model = mb._model(20, 3, dev)
    g = torch.Generator().manual_seed(3)
    B, Nc, Nt = 64, 2048, 256
    xs, ys = zip(*[mb._dataset(g, Nc + Nt, 20, 32, 0.1) for _ in range(B)])
    x, y = torch.stack(xs).to(dev), torch.stack(ys).to(dev)
    xc, yc, xt, yt = x[:, :Nc].contiguous(), y[:, :Nc].contiguous(), x[:, Nc:].contiguous(), y[:, Nc:].contiguous()
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
    import microbench as mb
    import ar_tabpfn
    dev = torch.device("cuda")
    model = mb._model(100, 4, dev)
    with torch.no_grad():
        model.ar_tokens.zero_()
    p = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="triton_shared_context", precision="bf16")
    g = torch.Generator().manual_seed(4)
    B, Nc, Nt = 256, 16384, 12
    x, y = mb._dataset(g, Nc + Nt, 100, 64, 0.05, product_frac=0.2)
    x, y = x.to(dev), y.to(dev)
    xc, yc = x[:Nc].expand(B, -1, -1), y[:Nc].expand(B, -1)
    xt = x[Nc:].expand(B, -1, -1).contiguous()
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
