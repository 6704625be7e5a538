"""The entry point that needs no caller scratch (artab_context_attention_noalloc).

Some hosts cannot allocate device memory when they call the library (a serving
arena sized up front, a plugin that only receives tensors).  For them the
split-context attention keeps its per-split partials in an array built into the
library.  This test calls it through the C ABI twice in a row, with different
inputs, and checks each result against the ordinary entry points fed with
caller-allocated partial buffers.  Collected last so that a failure here cannot
hide any other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_path(lib, _lib, code, q, k, v, rows, H, Dh, Nc, Ncp, splits):
    o = torch.empty(splits, rows, H, Dh, device=q.device)
    l = torch.empty(splits, rows, H, device=q.device)
    status = torch.zeros(1, dtype=torch.int32, device=q.device)
    out = torch.empty(rows, H, Dh, device=q.device)
    st = _lib.stream_ptr()
    _lib.check(lib.artab_context_attention(code, _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), rows, rows, 1, H, Dh, Nc,
                                           Ncp, splits, _lib.ptr(o), _lib.ptr(l), _lib.ptr(status), st))
    _lib.check(lib.artab_buffer_attention_merge(code, _lib.ptr(q), None, rows, H, Dh, 0, 0, 1, 0, _lib.ptr(o),
                                                _lib.ptr(l), splits, rows, _lib.ptr(out), st))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_matches_caller_scratch_twice(dtype):
    from ar_tabpfn import _lib
    from ar_tabpfn.model.triton_kernels import pack_context
    lib = _lib.lib()
    code = _lib.dtype_code(dtype)
    H, Dh = 4, 32
    g = torch.Generator(device="cuda").manual_seed(5)
    # calls in a row, each smaller than the one before: stale partials must not leak.  The last one asks
    # for more splits than the context has key tiles, so an empty split (zero output, -inf weight) goes
    # through the built-in array right after a larger call has filled it.
    for rows, Nc, splits in ((300, 1000, 4), (70, 260, 3), (40, 260, 4)):
        q = torch.randn(rows, H, Dh, device="cuda", generator=g).to(dtype)
        k = torch.randn(H, Nc, Dh, device="cuda", generator=g).to(dtype)
        v = torch.randn(H, Nc, Dh, device="cuda", generator=g).to(dtype)
        kp, vp, _, Ncp = pack_context(k, v)
        want = _reference_path(lib, _lib, code, q, kp, vp, rows, H, Dh, Nc, Ncp, splits)
        got = torch.empty(rows, H, Dh, device="cuda")
        _lib.check(lib.artab_context_attention_noalloc(code, _lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), rows, rows, 1, H,
                                                       Dh, Nc, Ncp, splits, _lib.ptr(got), _lib.stream_ptr()))
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)
        # and against plain fp32 attention, within the tolerance of the other operator tests
        s = torch.einsum("rhd,hnd->rhn", q.float(), k.float()) * Dh ** -0.5
        ref = torch.einsum("rhn,hnd->rhd", torch.softmax(s, -1), v.float())
        tol = 1e-5 if dtype == torch.float32 else 1e-2 * ref.abs().max().item()
        assert (got - ref).abs().max().item() <= tol


def test_no_alloc_rejects_oversized_requests():
    from ar_tabpfn import _lib
    lib = _lib.lib()
    q = torch.zeros(8, device="cuda")
    with pytest.raises(ValueError, match="built-in scratch"):
        _lib.check(lib.artab_context_attention_noalloc(_lib.F32, _lib.ptr(q), _lib.ptr(q), _lib.ptr(q), 100000, 100000,
                                                       1, 8, 32, 1024, 1024, 4, _lib.ptr(q), _lib.stream_ptr()))
