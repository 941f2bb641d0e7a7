"""Host-side logic of the dim_in-sharded mode on two CPU ranks (gloo): slicing, the reduction
operator per norm, and the combine of partial norms, checked against the unsharded oracle."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from oracle import bounds_oracle as O


def _partials(lw, uw, p):
    if p == 1:
        return lw.abs().amax(-2), uw.abs().amax(-2)
    if p == 2:
        return (lw * lw).sum(-2), (uw * uw).sum(-2)
    return lw.abs().sum(-2), uw.abs().sum(-2)


def _worker(rank, world, port, p, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from faith_b200 import sharded
        lw, lb, uw, ub = cases.rand_bounds(700, 2, 3, 23, 20, -0.7, 0.3)     # 23 rows: uneven split
        slw, suw = sharded.shard_bounds(lw, uw, rank, world)
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([slw.shape[-2]]))
        assert sum(int(s) for s in sizes) == 23
        pl, pu = _partials(slw, suw, p)
        nl, nu = sharded.reduce_partials(pl, pu, p)
        if p == 2:
            nl, nu = nl.sqrt(), nu.sqrt()
        l, u = lb - 0.5 * nl, ub + 0.5 * nu
        ol, ou = O.OBounds(p, 0.5, lw, lb, uw, ub).concretize()
        ok = torch.allclose(l, ol, rtol=1e-5, atol=1e-6) and torch.allclose(u, ou, rtol=1e-5, atol=1e-6)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("p", [1.0, 2.0, float("inf")])
def test_partial_norm_reduction_two_ranks(p):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + int(p if p < 10 else 7)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, p, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=120) for _ in procs]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert all(ok for _, ok in res)


def test_shard_bounds_covers_every_row_once():
    from faith_b200 import sharded
    lw = torch.arange(10.0).view(1, 1, 10, 1)
    for world in (1, 2, 3, 4, 8):
        parts = [sharded.shard_bounds(lw, lw, r, world)[0] for r in range(world)]
        assert torch.equal(torch.cat(parts, dim=-2), lw)
