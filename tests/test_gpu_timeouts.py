"""The give-up path of the bounded device-side waits, exercised without faulting anything: a
diagnostic switch makes the context contraction's MMA thread withhold its "scores ready" signal and
the wait limit is set to a fraction of a millisecond, so the softmax threads' waits run out, the
CTAs write nothing, free what they hold and the kernel returns normally with a non-zero status."""
import pytest
import torch

from util import ref_attention

pytestmark = pytest.mark.gpu


def _problem(rows=96, H=2, Nc=100, Dh=32):
    from ar_tabpfn.model import triton_kernels as tk
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(rows, H, Dh, device="cuda", generator=g).bfloat16()
    k = torch.randn(H, Nc, Dh, device="cuda", generator=g).bfloat16()
    v = torch.randn(H, Nc, Dh, device="cuda", generator=g).bfloat16()
    kp, vp, _, Ncp = tk.pack_context(k, v)
    return q, k, v, kp, vp, Ncp


def _ctx(lib, _lib, q, kp, vp, Nc, Ncp, out, lse, status, splits=1):
    rows, H, Dh = q.shape
    return lib.artab_context_attention(_lib.BF16, _lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), rows, rows, 1, H, Dh, Nc,
                                       Ncp, splits, _lib.ptr(out), _lib.ptr(lse), _lib.ptr(status),
                                       _lib.stream_ptr())


def test_wait_runs_out_status_is_set_and_the_next_launch_is_correct():
    from ar_tabpfn import _lib
    lib = _lib.lib()
    q, k, v, kp, vp, Ncp = _problem()
    rows, H, Dh = q.shape
    Nc = k.shape[1]
    out = torch.full((1, rows, H, Dh), -7.0, device="cuda")
    lse = torch.full((1, rows, H), -7.0, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    try:
        _lib.check(lib.artab_debug_set(_lib.DEBUG_WAIT_CYCLES, 200_000))       # ~0.1 ms
        _lib.check(lib.artab_debug_set(_lib.DEBUG_DROP_SCORE_COMMITS, 1))
        rc = _ctx(lib, _lib, q, kp, vp, Nc, Ncp, out, lse, status)
        torch.cuda.synchronize()
    finally:
        lib.artab_debug_set(_lib.DEBUG_DROP_SCORE_COMMITS, 0)
        lib.artab_debug_set(_lib.DEBUG_WAIT_CYCLES, 0)
    assert rc == 0                                   # the launch itself succeeded ...
    assert int(status.item()) != 0                   # ... the kernel reports that a wait gave up ...
    assert bool((out == -7.0).all()) and bool((lse == -7.0).all())   # ... and wrote no result
    # the context is intact: the same call without the switch is correct
    status.zero_()
    _lib.check(_ctx(lib, _lib, q, kp, vp, Nc, Ncp, out, lse, status))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want, want_lse = ref_attention(q.permute(1, 0, 2).unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0))
    got = out[0].permute(1, 0, 2).unsqueeze(0)
    assert float((got - want).abs().max() / want.abs().max()) <= 1e-2
    torch.testing.assert_close(lse[0].t().unsqueeze(0), want_lse, atol=2e-3, rtol=0)


def test_noalloc_entry_reports_a_timed_out_wait_as_nan():
    from ar_tabpfn import _lib
    lib = _lib.lib()
    q, k, v, kp, vp, Ncp = _problem(rows=64, Nc=300)
    rows, H, Dh = q.shape
    Nc = k.shape[1]
    out = torch.zeros(rows, H, Dh, device="cuda")

    def call():
        return lib.artab_context_attention_noalloc(_lib.BF16, _lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), rows, rows, 1,
                                                   H, Dh, Nc, Ncp, 2, _lib.ptr(out), _lib.stream_ptr())
    _lib.check(call())       # also the one-off look-up of the built-in array, outside the failing call
    torch.cuda.synchronize()
    good = out.clone()
    try:
        _lib.check(lib.artab_debug_set(_lib.DEBUG_WAIT_CYCLES, 200_000))
        _lib.check(lib.artab_debug_set(_lib.DEBUG_DROP_SCORE_COMMITS, 1))
        rc = call()
        torch.cuda.synchronize()
    finally:
        lib.artab_debug_set(_lib.DEBUG_DROP_SCORE_COMMITS, 0)
        lib.artab_debug_set(_lib.DEBUG_WAIT_CYCLES, 0)
    assert rc == 0 and bool(torch.isnan(out).all())   # never a plausible mix of stale partials
    _lib.check(call())
    torch.cuda.synchronize()
    assert torch.equal(out, good)


def test_predictor_raises_after_a_timed_out_call():
    from ar_tabpfn import _lib
    from ar_tabpfn.model import ARTabPFNPredictor
    import synthetic as syn
    lib = _lib.lib()
    m = syn.build_model(6, 9, d_model=64, n_heads=2, n_layers=2, d_ff=256).cuda()
    p = ARTabPFNPredictor.from_trained_model(m, backend="triton_shared_context", precision="bf16")
    g = torch.Generator(device="cuda").manual_seed(1)
    xc, yc = torch.randn(4, 40, 6, device="cuda", generator=g), torch.randn(4, 40, device="cuda", generator=g)
    xt, yt = torch.randn(4, 5, 6, device="cuda", generator=g), torch.randn(4, 5, device="cuda", generator=g)
    good = p.evaluate_joint_density(xc, yc, xt, yt).clone()
    assert p.last_status() == 0
    try:
        _lib.check(lib.artab_debug_set(_lib.DEBUG_WAIT_CYCLES, 200_000))
        _lib.check(lib.artab_debug_set(_lib.DEBUG_DROP_SCORE_COMMITS, 1))
        p.evaluate_joint_density(xc, yc, xt, yt)
        torch.cuda.synchronize()
    finally:
        lib.artab_debug_set(_lib.DEBUG_DROP_SCORE_COMMITS, 0)
        lib.artab_debug_set(_lib.DEBUG_WAIT_CYCLES, 0)
    assert p.last_status() != 0
    with pytest.raises(_lib.ArtabError, match="wait gave up"):
        p.evaluate_joint_density(xc, yc, xt, yt)
    # the error is reported once; the predictor then works again
    assert torch.equal(p.evaluate_joint_density(xc, yc, xt, yt), good)
    assert p.last_status() == 0
