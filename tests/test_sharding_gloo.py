"""World-size-2 gloo test of the stream sharding (host logic of the multi-GPU path).

The per-rank work is the CPU oracle here (the shipped kernels need a GPU); what is
under test is the partition, the variate slicing and the gather: the sharded result
must equal the single-process result exactly.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmp):
    for p in (os.path.join(ROOT, "ar-nanotabpfn_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import artab_oracle as orc
    from ar_tabpfn.sharding import sharded_call
    from util import load_golden
    fx = load_golden("tiny_distinct.pt")

    def run(xc, yc, xt, expo, normal):
        y, ld, _ = orc.OraclePredictor(fx["state_dict"], fx["n_heads"]).sample_sequence(
            xc, yc, xt, expo, normal, shared=False)
        return y, ld

    y, ld = sharded_call(run, (fx["xc"], fx["yc"], fx["xt"]), (fx["expo"], fx["normal"]))
    if rank == 0:
        torch.save((y, ld), tmp)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    from ar_tabpfn.sharding import shard_bounds
    for n in (1, 3, 7, 8, 512, 4096):
        for w in (1, 2, 3, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= 1


@pytest.mark.timeout(300)
def test_two_rank_gloo_matches_single_process(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import artab_oracle as orc
    from util import load_golden
    fx = load_golden("tiny_distinct.pt")     # 3 streams over 2 ranks: uneven split
    want_y, want_ld, _ = orc.OraclePredictor(fx["state_dict"], fx["n_heads"]).sample_sequence(
        fx["xc"], fx["yc"], fx["xt"], fx["expo"], fx["normal"], shared=False)
    out = str(tmp_path / "gathered.pt")
    mp.spawn(_worker, args=(2, 29500 + os.getpid() % 2000, out), nprocs=2, join=True)
    y, ld = torch.load(out)
    torch.testing.assert_close(y, want_y, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(ld, want_ld, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(y, fx["samples_flex"], atol=1e-5, rtol=1e-5)
