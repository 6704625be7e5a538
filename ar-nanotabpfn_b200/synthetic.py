"""Seeded synthetic models and datasets of the benchmark configurations.

One place for what the benchmark, the micro-benchmarks and the tests must agree on: the same
model weights and the same rows, so that a parity test checks exactly what a benchmark times.
No public dataset is involved anywhere; every input is drawn here from a seeded generator with
the shapes and value distributions of the named configuration:

  config 3  6 layers, d_model 192, 6 heads, MLP 768; one dataset of 1024 context rows x 20
            features; 128 targets decoded by 512 sample streams sharing the context; seed 2
  config 4  same model; 64 independent datasets of 2048 context rows + 256 targets; seed 3
  config 5  same model with 100 features (20 % of the columns pairwise products), tanh-MLP
            100-64-64-1 labels with noise 0.05; 16384 context rows, 256 targets, 4096 streams;
            seed 4

Weights: reference defaults + Xavier-uniform on every nn.Linear weight, then rounded to
bf16-representable values (the bf16-mode protocol: the fp32 oracle runs on the same rounded
weights and inputs).
"""
from __future__ import annotations

import torch

MODEL_6L = dict(d_model=192, n_heads=6, n_layers=6, d_ff=768, buffer_size=8, num_components=5)

CONFIG3 = dict(seed=2, num_features=20, n_ctx=1024, n_targets=128, streams=512, hidden=32, noise=0.1)
CONFIG4 = dict(seed=3, num_features=20, n_ctx=2048, n_targets=256, datasets=64, hidden=32, noise=0.1)
CONFIG5 = dict(seed=4, num_features=100, n_ctx=16384, n_targets=256, streams=4096, hidden=64, noise=0.05,
               product_frac=0.2)


def build_model(num_features: int, seed: int, bf16_round: bool = True, **overrides):
    """The 6-layer benchmark model (on the CPU; move it with ``.to(device)``)."""
    import ar_tabpfn
    cfg = dict(MODEL_6L, num_features=num_features)
    cfg.update(overrides)
    torch.manual_seed(seed)
    m = ar_tabpfn.ARTabPFN(**cfg).eval()
    with torch.no_grad():
        for mod in m.modules():
            if isinstance(mod, torch.nn.Linear):
                torch.nn.init.xavier_uniform_(mod.weight)
        for p in m.parameters():
            if bf16_round:
                p.copy_(p.to(torch.bfloat16).float())
            p.requires_grad_(False)
    return m


def dataset(g: torch.Generator, n_rows: int, n_feat: int, hidden: int = 32, noise: float = 0.1,
            product_frac: float = 0.0):
    """x ~ N(0,1) (optionally a fraction of the columns replaced by products of two others),
    standardised per column; y = tanh-MLP(F -> hidden -> hidden -> 1) + N(0, noise^2)."""
    x = torch.randn(n_rows, n_feat, generator=g)
    n_prod = int(product_frac * n_feat)
    for j in range(n_prod):
        a, b = torch.randint(n_prod, n_feat, (2,), generator=g).tolist()
        x[:, j] = x[:, a] * x[:, b]
    x = (x - x.mean(0)) / x.std(0)
    w1 = torch.randn(n_feat, hidden, generator=g) / n_feat ** 0.5
    w2 = torch.randn(hidden, hidden, generator=g) / hidden ** 0.5
    w3 = torch.randn(hidden, 1, generator=g) / hidden ** 0.5
    y = (torch.tanh(torch.tanh(x @ w1) @ w2) @ w3)[:, 0] + noise * torch.randn(n_rows, generator=g)
    return x, y


def _bf16(t):
    return t.to(torch.bfloat16).float()


def config3_model():
    return build_model(CONFIG3["num_features"], CONFIG3["seed"])


def config3_rows(n_targets: int = None):
    """(x_context [Nc,F], y_context [Nc], x_target [Nt,F], y_target [Nt]) of the one dataset,
    bf16-representable."""
    c = CONFIG3
    nt = c["n_targets"] if n_targets is None else n_targets
    g = torch.Generator().manual_seed(c["seed"])
    x, y = dataset(g, c["n_ctx"] + c["n_targets"], c["num_features"], c["hidden"], c["noise"])
    x, y = _bf16(x), _bf16(y)
    nc = c["n_ctx"]
    return x[:nc], y[:nc], x[nc:nc + nt], y[nc:nc + nt]


def config3_workload(streams: int, n_targets: int = None):
    """Batched inputs of config 3: the dataset repeated over the sample streams."""
    xc, yc, xt, _ = config3_rows(n_targets)
    return (xc.expand(streams, -1, -1).contiguous(), yc.expand(streams, -1).contiguous(),
            xt.expand(streams, -1, -1).contiguous())


def variates(seed: int, n_steps: int, streams: int, n_comp: int, device):
    """Full-job random numbers in the order the sampler consumes them (all Exp(1) [Nt,B,K], then
    all N(0,1) [Nt,B]) from a seeded generator on ``device``."""
    g = torch.Generator(device=device).manual_seed(seed)
    expo = torch.empty(n_steps, streams, n_comp, device=device).exponential_(1.0, generator=g)
    normal = torch.randn(n_steps, streams, device=device, generator=g)
    return expo, normal


def config4_model():
    return build_model(CONFIG4["num_features"], CONFIG4["seed"])


def config4_workload(datasets: int = None, n_ctx: int = None, n_targets: int = None):
    """(xc [B,Nc,F], yc [B,Nc], xt [B,Nt,F], yt [B,Nt]): independent datasets."""
    c = CONFIG4
    B = c["datasets"] if datasets is None else datasets
    nc = c["n_ctx"] if n_ctx is None else n_ctx
    nt = c["n_targets"] if n_targets is None else n_targets
    g = torch.Generator().manual_seed(c["seed"])
    xs, ys = zip(*[dataset(g, nc + nt, c["num_features"], c["hidden"], c["noise"]) for _ in range(B)])
    x, y = _bf16(torch.stack(xs)), _bf16(torch.stack(ys))
    return x[:, :nc].contiguous(), y[:, :nc].contiguous(), x[:, nc:].contiguous(), y[:, nc:].contiguous()


def config5_model():
    return build_model(CONFIG5["num_features"], CONFIG5["seed"])


def config5_rows(n_ctx: int = None, n_targets: int = None):
    """(x_context [Nc,F], y_context [Nc], x_target [Nt,F], y_target [Nt]) of the one dataset."""
    c = CONFIG5
    nc = c["n_ctx"] if n_ctx is None else n_ctx
    nt = c["n_targets"] if n_targets is None else n_targets
    g = torch.Generator().manual_seed(c["seed"])
    x, y = dataset(g, nc + nt, c["num_features"], c["hidden"], c["noise"], c["product_frac"])
    x, y = _bf16(x), _bf16(y)
    return x[:nc], y[:nc], x[nc:], y[nc:]
