"""The C-ABI library: builds, loads and exports every symbol include/artab.h declares
(no compute call is made; runs without a GPU)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "artab.h")).read()
    return sorted(set(re.findall(r"ARTAB_API[^;(]*?\b(artab_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for s in ("artab_prefill", "artab_decode_step", "artab_teacher_forcing", "artab_context_attention",
              "artab_buffer_attention_merge", "artab_kv_append", "artab_embed", "artab_head_sample",
              "artab_head_logpdf"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as ge
    ge.build()
    from ar_tabpfn import _lib
    lib = _lib.load_library()
    for s in declared_symbols():
        assert hasattr(lib, s), s
        assert s in _lib._SIGNATURES, f"{s} has no ctypes signature"
    assert lib.artab_version().startswith(b"artab-b200")
    assert lib.artab_last_error() is not None
    lib.artab_launch_count_reset()
    assert lib.artab_launch_count() == 0


def test_product_fails_loudly_without_cuda():
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from ar_tabpfn import _lib
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()
    import ar_tabpfn
    m = ar_tabpfn.ARTabPFN(d_model=32, n_heads=2, n_layers=1, d_ff=64, num_features=3)
    p = ar_tabpfn.ARTabPFNPredictor.from_trained_model(m)
    with pytest.raises(RuntimeError):
        p.sample_sequence(torch.zeros(1, 4, 3), torch.zeros(1, 4), torch.zeros(1, 2, 3))


def test_state_dict_is_reference_compatible():
    """Reference checkpoints load unchanged: same keys and shapes as the golden state_dict."""
    import torch
    import ar_tabpfn
    fx = torch.load(os.path.join(ROOT, "tests", "golden", "config1.pt"), weights_only=False)
    m = ar_tabpfn.ARTabPFN(**fx["cfg"])
    own = m.state_dict()
    assert set(own) == set(fx["state_dict"])
    for k, v in fx["state_dict"].items():
        assert own[k].shape == v.shape, k


def test_checkpoint_of_the_training_script_loads(tmp_path):
    """{"step", "model"} files whose embedder / head keys carry torch.compile's ``_orig_mod.``
    prefix load into the drop-in model with every size read from the shapes (host logic only)."""
    import torch
    import ar_tabpfn
    src = ar_tabpfn.ARTabPFN(d_model=64, n_heads=4, n_layers=3, d_ff=128, num_features=10, buffer_size=32,
                             num_components=20)
    sd = {}
    for k, v in src.state_dict().items():
        head, _, rest = k.partition(".")
        sd[f"{head}._orig_mod.{rest}" if head in ("embedder", "head") else k] = v.clone()
    path = tmp_path / "step_10.pt"
    torch.save({"step": 10, "model": sd}, path)
    m = ar_tabpfn.ARTabPFN.from_checkpoint(str(path), n_heads=4)
    assert (m.d_model, m.buffer_size, len(m.backbone.layers), m.head.num_components) == (64, 32, 3, 20)
    for k, v in src.state_dict().items():
        assert torch.equal(m.state_dict()[k], v)
    assert not m.training
    import pytest
    with pytest.raises(ValueError):
        ar_tabpfn.ARTabPFN.from_checkpoint(sd, n_heads=5)
