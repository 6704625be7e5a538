"""Generate the golden fixtures in this directory from the real reference.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference [--forward-only | --ragged-only | --columns-only]

It imports the reference's ``ar_tabpfn.model`` package under the alias
``ref_ar_tabpfn`` (so it cannot collide with the shipped drop-in package of
the same name), runs the reference on CPU in fp32 under ``torch.no_grad`` and
stores inputs, weights and outputs as small ``.pt`` files.  The test-suite
only ever reads the stored files.
"""

from __future__ import annotations

import importlib
import importlib.util
import math
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import artab_oracle as orc  # noqa: E402  (data generators + variate order only)


def import_reference(root: str):
    pkg = types.ModuleType("ref_ar_tabpfn")
    pkg.__path__ = [os.path.join(root, "ar_tabpfn")]
    sys.modules["ref_ar_tabpfn"] = pkg
    return importlib.import_module("ref_ar_tabpfn.model"), importlib.import_module(
        "ref_ar_tabpfn.model.triton_kernels")


def xavier_model(ref, seed, **kw):
    """Small CPU-sized model of the first benchmark configuration: reference defaults + Xavier-uniform on
    every nn.Linear weight."""
    torch.manual_seed(seed)
    m = ref.ARTabPFN(**kw).eval()
    for mod in m.modules():
        if isinstance(mod, torch.nn.Linear):
            torch.nn.init.xavier_uniform_(mod.weight)
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def sd_of(m):
    return {k: v.detach().clone() for k, v in m.state_dict().items()}


@torch.no_grad()
def ops_fixture(tk):
    """Known-answer vectors of the functional attention operators, shapes
    taken from the reference's own unit tests (non-divisible batch 37,
    context 100, Lq in {1,2,5}, empty buffer, all-masked first target row)."""
    g = torch.Generator().manual_seed(42)
    out = {}

    def rn(*s):
        return torch.randn(*s, generator=g)

    cases = []
    for (B, H, Lq, Nc, Dh, Nb) in [(37, 4, 1, 64, 32, 5), (32, 4, 1, 100, 32, 0), (8, 2, 5, 33, 16, 7),
                                   (3, 4, 2, 128, 32, 63), (16, 8, 1, 96, 64, 1)]:
        q, k, v = rn(B, H, Lq, Dh), rn(H, Nc, Dh), rn(H, Nc, Dh)
        kb, vb = rn(B, H, Nb, Dh), rn(B, H, Nb, Dh)
        o_c, l_c = tk.pytorch_context_attention(q, k, v)
        case = dict(q=q, k_ctx=k, v_ctx=v, k_buf=kb, v_buf=vb, out_ctx=o_c, lse_ctx=l_c,
                    hybrid=tk.hybrid_attention(q, k, v, kb, vb, use_triton=False))
        if Nb > 0:
            o_b, l_b = tk.pytorch_buffer_attention(q, kb, vb)
            case.update(out_buf=o_b, lse_buf=l_b, merged=tk.merge_attention_outputs(o_c, l_c, o_b, l_b))
        cases.append(case)
    out["attn"] = cases

    tf = []
    for (B, H, Nt, Nc, Dh) in [(2, 4, 4, 16, 32), (3, 2, 9, 40, 16)]:
        q, k, v = rn(B, H, 2 * Nt, Dh), rn(H, Nc, Dh), rn(H, Nc, Dh)
        kb, vb = rn(B, H, Nt, Dh), rn(B, H, Nt, Dh)
        o_b, l_b = tk.pytorch_teacher_forcing_buffer_attention(q, kb, vb, num_targets=Nt)
        tf.append(dict(q=q, k_ctx=k, v_ctx=v, k_buf=kb, v_buf=vb, num_targets=Nt,
                       mask=tk._teacher_forcing_buffer_mask(Nt, q.device).clone(),
                       out_buf=o_b, lse_buf=l_b,
                       hybrid=tk.hybrid_teacher_forcing_attention(q, k, v, kb, vb, Nt, use_triton=False)))
    out["tf"] = tf
    return out


@torch.no_grad()
def run_reference_sampling(ref, model, xc, yc, xt, seed, backend):
    """Reference sample_sequence with torch's global CPU generator seeded, also
    recording the per-step target representation so that the log density of
    each drawn value can be evaluated with the reference head."""
    pred = ref.ARTabPFNPredictor.from_trained_model(model, backend=backend)
    zs = []
    orig = model.head.sample

    def spy(z, num_samples=1):
        zs.append(z.clone())
        return orig(z, num_samples)

    model.head.sample = spy
    try:
        torch.manual_seed(seed)
        ys = pred.sample_sequence(xc, yc, xt)
    finally:
        del model.head.sample
    z = torch.cat(zs, dim=1)                                  # [B,Nt,D]
    ld = model.head.log_likelihood(z, ys.unsqueeze(-1))       # [B,Nt]
    ctx = None
    if backend == "triton_shared_context":
        ctx = [(l.k_ctx_cache.clone(), l.v_ctx_cache.clone()) for l in model.backbone.layers]
    return ys, ld, z, ctx


@torch.no_grad()
def model_fixture(ref, name, seed, cfg, Nc, Nt, B, shared_data, variate_seed):
    m = xavier_model(ref, seed, **cfg)
    F = cfg["num_features"]
    if shared_data:
        x, y = orc.make_dataset(seed, Nc + Nt, F)
        xc, yc = x[:Nc].expand(B, -1, -1).contiguous(), y[:Nc].expand(B, -1).contiguous()
        xt, yt = x[Nc:].expand(B, -1, -1).contiguous(), y[Nc:].expand(B, -1).contiguous()
    else:
        ds = [orc.make_dataset(seed * 1000 + b, Nc + Nt, F) for b in range(B)]
        xc = torch.stack([d[0][:Nc] for d in ds]); yc = torch.stack([d[1][:Nc] for d in ds])
        xt = torch.stack([d[0][Nc:] for d in ds]); yt = torch.stack([d[1][Nc:] for d in ds])
    fx = dict(name=name, cfg=cfg, n_heads=cfg["n_heads"], state_dict=sd_of(m), xc=xc, yc=yc, xt=xt, yt=yt,
              variate_seed=variate_seed)
    K = cfg["num_components"]
    expo, normal = orc.draw_variates(variate_seed, Nt, B, K)
    fx["expo"], fx["normal"] = expo, normal
    for be, tag in (("triton_shared_context", "shared"), ("flex_attention", "flex")):
        ys, ld, z, ctx = run_reference_sampling(ref, m, xc, yc, xt, variate_seed, be)
        fx[f"samples_{tag}"], fx[f"sample_logdens_{tag}"], fx[f"z_{tag}"] = ys, ld, z
        if ctx is not None:
            fx["ctx_kv"] = ctx
        pred = ref.ARTabPFNPredictor.from_trained_model(m, backend=be)
        fx[f"joint_logdens_{tag}"] = pred.evaluate_joint_density(xc, yc, xt, yt)
    return fx


@torch.no_grad()
def forward_fixture(ref, root):
    """The training forward (ARTabPFN.forward under create_row_mask) run for inference: the
    scalar loss the reference returns plus the per-target log density and representation,
    captured at the head.  Case "tf_style" uses the inference-style mask of the reference's
    own test_teacher_forcing_matches_forward (buffer j sees buffers <= j, target i sees
    buffers < i), built with the same flex primitives."""
    attn = importlib.import_module("ref_ar_tabpfn.model.attention")
    from torch.nn.attention.flex_attention import create_block_mask
    cases = []
    specs = [
        dict(name="default_chunks", seed=21, B=3, Nc=10, Nb=4, Nt=16, chunks=None,
             cfg=dict(d_model=32, n_heads=2, n_layers=2, d_ff=64, num_features=4, buffer_size=4, num_components=3)),
        dict(name="dh32_three_chunks", seed=5, B=4, Nc=50, Nb=8, Nt=32, chunks=3,
             cfg=dict(d_model=64, n_heads=2, n_layers=3, d_ff=128, num_features=5, buffer_size=8, num_components=5)),
        dict(name="short_buffer", seed=23, B=2, Nc=33, Nb=3, Nt=12, chunks=None,
             cfg=dict(d_model=64, n_heads=4, n_layers=2, d_ff=128, num_features=8, buffer_size=8, num_components=5)),
        dict(name="tf_style", seed=24, B=2, Nc=8, Nb=4, Nt=4, chunks="tf",
             cfg=dict(d_model=32, n_heads=2, n_layers=2, d_ff=64, num_features=4, buffer_size=4, num_components=3)),
    ]
    for sp in specs:
        m = xavier_model(ref, sp["seed"], **sp["cfg"])
        B, Nc, Nb, Nt, F = sp["B"], sp["Nc"], sp["Nb"], sp["Nt"], sp["cfg"]["num_features"]
        ds = [orc.make_dataset(sp["seed"] * 1000 + b, Nc + Nb + Nt, F) for b in range(B)]   # one dataset per element
        x, y = torch.stack([d[0] for d in ds]), torch.stack([d[1] for d in ds])
        xc, yc = x[:, :Nc].contiguous(), y[:, :Nc].contiguous()
        xb, yb = x[:, Nc:Nc + Nb].contiguous(), y[:, Nc:Nc + Nb].contiguous()
        xt, yt = x[:, Nc + Nb:].contiguous(), y[:, Nc + Nb:].contiguous()
        R = Nc + Nb + Nt
        attn.clear_mask_cache()
        mf = attn.create_dense_mask(seq_len=1, device="cpu")
        if sp["chunks"] == "tf":
            def mask_mod(b, h, q_idx, kv_idx, Nc=Nc, Nb=Nb):
                ctx = kv_idx < Nc
                kv_buf = (kv_idx >= Nc) & (kv_idx < Nc + Nb)
                q_buf = (q_idx >= Nc) & (q_idx < Nc + Nb)
                q_tgt = q_idx >= Nc + Nb
                return ctx | (q_buf & kv_buf & (kv_idx <= q_idx)) | (q_tgt & kv_buf & ((kv_idx - Nc) < (q_idx - Nc - Nb)))
            mr = create_block_mask(mask_mod, B=None, H=None, Q_LEN=R, KV_LEN=R, device="cpu")
            visible = [j + 1 for j in range(Nb)] + list(range(Nt))
        else:
            mr = attn.create_row_mask(num_rows=R, context_len=Nc, buffer_len=Nb, attending_chunks=sp["chunks"],
                                      device="cpu")
            visible = orc.row_mask_visible(Nb, Nt, sp["chunks"])
        zs = []
        orig = m.head.forward

        def spy(z, y=None, loss_mask=None):
            zs.append(z.clone())
            return orig(z, y, loss_mask)

        m.head.forward = spy
        try:
            loss = m(x_context=xc, y_context=yc, x_buffer=xb, y_buffer=yb, x_target=xt, mask_features=mf,
                     mask_rows=mr, y_target=yt)
        finally:
            del m.head.forward
        z = zs[0]
        ld = m.head.log_likelihood(z, yt.unsqueeze(-1))
        cases.append(dict(name=sp["name"], cfg=sp["cfg"], n_heads=sp["cfg"]["n_heads"], state_dict=sd_of(m),
                          xc=xc, yc=yc, xb=xb, yb=yb, xt=xt, yt=yt, attending_chunks=sp["chunks"],
                          visible=visible, loss=loss.clone(), logdens=ld, z=z))
    return cases


@torch.no_grad()
def ragged_fixture(tk):
    """Ragged private buffers: the reference's masked buffer attention and hybrid attention with
    one visible prefix per stream (lengths include 0 = nothing visible and the full buffer)."""
    g = torch.Generator().manual_seed(77)
    cases = []
    for (B, H, Lq, Nc, Dh, Nb) in [(9, 4, 1, 64, 32, 12), (5, 2, 2, 40, 16, 7), (6, 3, 1, 33, 64, 20),
                                   (16, 4, 2, 128, 32, 63)]:
        rn = lambda *s: torch.randn(*s, generator=g)
        q, k, v = rn(B, H, Lq, Dh), rn(H, Nc, Dh), rn(H, Nc, Dh)
        kb, vb = rn(B, H, Nb, Dh), rn(B, H, Nb, Dh)
        lens = torch.randint(0, Nb + 1, (B,), generator=g)
        lens[0], lens[-1] = 0, Nb
        mask = (torch.arange(Nb)[None, :] < lens[:, None])[:, None, None, :].expand(B, H, Lq, Nb).contiguous()
        o_b, l_b = tk.pytorch_buffer_attention(q, kb, vb, mask=mask)
        cases.append(dict(q=q, k_ctx=k, v_ctx=v, k_buf=kb, v_buf=vb, lens=lens, mask=mask, out_buf=o_b, lse_buf=l_b,
                          hybrid=tk.hybrid_attention(q, k, v, kb, vb, buf_mask=mask, use_triton=False)))
    return cases


@torch.no_grad()
def columns_fixture(ref, root):
    """The reference's backbone (TwoStageTransformer) on inputs with SEVERAL column tokens per row,
    x [B, R, C, D] with C > 1: feature attention across the C tokens of a row under
    create_dense_mask(C), row attention over the R rows of every column under create_row_mask.
    Stored: input, weights, the output after the final norm and the row-attention K / V of layer 0."""
    attn = importlib.import_module("ref_ar_tabpfn.model.attention")
    cases = []
    for seed, (D, H, L, Dff, B, C, Nc, Nb, Nt) in enumerate([(64, 4, 2, 128, 2, 3, 20, 4, 8), (64, 2, 1, 128, 3, 5, 33, 2, 4),
                                                              (32, 2, 1, 64, 1, 2, 7, 1, 3)]):
        torch.manual_seed(100 + seed)
        m = ref.TwoStageTransformer(D, H, L, Dff).eval()
        for mod in m.modules():
            if isinstance(mod, torch.nn.Linear):
                torch.nn.init.xavier_uniform_(mod.weight)
        R = Nc + Nb + Nt
        x = torch.randn(B, R, C, D)
        mf = attn.create_dense_mask(C, device="cpu")
        mr = attn.create_row_mask(R, context_len=Nc, buffer_len=Nb, attending_chunks=1, device="cpu")
        out, kv = m(x, mf, mr)
        cases.append(dict(cfg=dict(d_model=D, n_heads=H, n_layers=L, d_ff=Dff), B=B, C=C, Nc=Nc, Nb=Nb, Nt=Nt,
                          attending_chunks=1, x=x, state_dict=sd_of(m), out=out, k0=kv[0][0], v0=kv[0][1]))
    return cases


def compact(o):
    """Clone every tensor so that no view drags a larger storage into the file."""
    if isinstance(o, torch.Tensor):
        return o.detach().clone().contiguous()
    if isinstance(o, dict):
        return {k: compact(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(compact(v) for v in o)
    return o


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    root = sys.argv[1]
    ref, tk = import_reference(root)
    torch.set_num_threads(8)
    if "--ragged-only" in sys.argv[2:]:       # leaves the other fixtures as they are
        torch.save(compact(ragged_fixture(tk)), os.path.join(HERE, "ragged.pt"))
        print("ragged.pt", os.path.getsize(os.path.join(HERE, "ragged.pt")))
        return
    if "--columns-only" in sys.argv[2:]:      # leaves the other fixtures as they are
        torch.save(compact(columns_fixture(ref, root)), os.path.join(HERE, "columns.pt"))
        print("columns.pt", os.path.getsize(os.path.join(HERE, "columns.pt")))
        return
    if "--forward-only" in sys.argv[2:]:      # leaves the other fixtures as they are
        torch.save(compact(forward_fixture(ref, root)), os.path.join(HERE, "forward.pt"))
        print("forward.pt", os.path.getsize(os.path.join(HERE, "forward.pt")))
        return
    torch.save(compact(ops_fixture(tk)), os.path.join(HERE, "ops.pt"))
    c1 = model_fixture(
        ref, "config1", seed=0,
        cfg=dict(d_model=64, n_heads=4, n_layers=2, d_ff=128, num_features=8, buffer_size=8, num_components=5),
        Nc=128, Nt=16, B=8, shared_data=True, variate_seed=0)
    torch.save(compact(c1), os.path.join(HERE, "config1.pt"))
    tiny = model_fixture(
        ref, "tiny_distinct", seed=42,
        cfg=dict(d_model=32, n_heads=2, n_layers=2, d_ff=64, num_features=4, buffer_size=4, num_components=3),
        Nc=8, Nt=11, B=3, shared_data=False, variate_seed=7)
    torch.save(compact(tiny), os.path.join(HERE, "tiny_distinct.pt"))
    # Dh = 32 model (the head size the bf16 tensor-core kernels are built for)
    h32 = model_fixture(
        ref, "dh32", seed=5,
        cfg=dict(d_model=64, n_heads=2, n_layers=3, d_ff=128, num_features=5, buffer_size=8, num_components=5),
        Nc=200, Nt=12, B=6, shared_data=True, variate_seed=11)
    torch.save(compact(h32), os.path.join(HERE, "dh32.pt"))
    torch.save(compact(forward_fixture(ref, root)), os.path.join(HERE, "forward.pt"))
    torch.save(compact(ragged_fixture(tk)), os.path.join(HERE, "ragged.pt"))
    torch.save(compact(columns_fixture(ref, root)), os.path.join(HERE, "columns.pt"))
    for f in ("ops.pt", "config1.pt", "tiny_distinct.pt", "dh32.pt", "forward.pt", "ragged.pt", "columns.pt"):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
