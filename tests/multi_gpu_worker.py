"""One rank of the multi-GPU tests (started by tests/test_gpu_multi.py, one process per GPU).

argv: rank world port case.  The process group (gloo) only carries the NCCL id and the pass or fail of each rank; all data-path
traffic goes through the library's communicator.  Prints "RANK r OK" when its checks hold."""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, HERE)


def main():
    rank, world, port, case = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", port
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import cases
    import helpers
    from faith_b200 import _lib, ops, sharded
    from faith_b200.comm import ALGO_NCCL, ALGO_ONESHOT, MAX, SUM, Comm
    from oracle import bounds_oracle as O
    comm = Comm.from_process_group(oneshot_floats=1 << 16)

    if case == "allreduce":
        for n in (1, 7, 1000, 40000, 1 << 16):
            g = torch.Generator().manual_seed(100 + n)
            parts = [torch.randn(n, generator=g) for _ in range(world)]
            for op, ref in ((SUM, sum(parts[1:], parts[0].clone())), (MAX, torch.stack(parts).amax(0))):
                outs = []
                for algo in (ALGO_NCCL, ALGO_ONESHOT):
                    for _ in range(3):                       # repeated calls alternate the slot sets
                        buf = parts[rank].clone().to(dev)
                        comm.all_reduce(buf, op, algo)
                    outs.append(buf.cpu())
                for o in outs:
                    assert torch.allclose(o, ref, rtol=1e-6, atol=1e-6), (n, op)
                # the one-shot sum adds in rank order on every rank: all ranks hold the same bits
                gathered = [torch.empty(n) for _ in range(world)]
                dist.all_gather(gathered, outs[1])
                assert all(torch.equal(gathered[0], t) for t in gathered)
        comm.check(sync=True)
    elif case == "relu":
        for p in (1.0, 2.0, float("inf")):
            lw, lb, uw, ub = cases.rand_bounds(801, 2, 3, 50, 36, -0.7, 0.2)
            slw, suw = sharded.shard_bounds(lw.to(dev), uw.to(dev), rank, world)
            ref = O.OBounds(p, 0.5, lw, lb, uw, ub).relu()
            rlw, ruw = sharded.shard_bounds(ref.lw, ref.uw, rank, world)
            for algo in (ALGO_NCCL, ALGO_ONESHOT):
                o = sharded.relax_sharded(_lib.FB_RELU, slw, suw, lb.to(dev), ub.to(dev), p, 0.5, comm=comm, algo=algo)
                helpers.assert_close(o[0], rlw, "lw")
                helpers.assert_close(o[1], ruw, "uw")
                helpers.assert_close(o[2], ref.lb, "lb")
                helpers.assert_close(o[3], ref.ub, "ub")
                l, u = sharded.concretize_sharded(slw, suw, lb.to(dev), ub.to(dev), p, 0.5, comm, algo)
                rl, ru = O.OBounds(p, 0.5, lw, lb, uw, ub).concretize()
                helpers.assert_close(l, rl, "l")
                helpers.assert_close(u, ru, "u")
        comm.check(sync=True)
    elif case == "cnn":
        layers = O.make_cnn(5, c_in=3, hw=8)
        img = torch.rand(3, 8, 8, generator=torch.Generator().manual_seed(5))
        ol, ou = O.cnn_forward(layers, img, float("inf"), 2.0 / 255)
        l64, u64 = O.cnn_forward([tuple(t.double() if isinstance(t, torch.Tensor) else t for t in ly) for ly in layers],
                                 img.double(), float("inf"), 2.0 / 255)
        for algo in (ALGO_NCCL, ALGO_ONESHOT):
            l, u = sharded.CnnVerifier(layers, dev, comm=comm, algo=algo).forward(img, float("inf"), 2.0 / 255, rank, world)
            helpers.assert_within_noise(l, ol, l64, "l")
            helpers.assert_within_noise(u, ou, u64, "u")
        comm.check(sync=True)
    elif case == "timeout":
        # rank 0 enters a one-shot all-reduce that nobody joins: its wait must run out (0.2 s), the kernel must return
        # and the check must report FB_ERR_TIMEOUT; the device stays usable.  The other ranks sit at the barrier below
        # with nothing in flight.
        if rank == 0:
            comm.set_wait_ns(200_000_000)
            buf = torch.ones(1000, device=dev)
            comm.all_reduce(buf, SUM, ALGO_ONESHOT)
            try:
                comm.check(sync=True)
                raise SystemExit("the expired wait was not reported")
            except _lib.FaithError as e:
                assert "expired" in str(e), str(e)
            assert float((torch.ones(10, device=dev) * 2).sum()) == 20.0
        dist.barrier()
    else:
        raise SystemExit("unknown case " + case)
    dist.barrier()
    comm.destroy()
    dist.destroy_process_group()
    print("RANK %d OK" % rank)


if __name__ == "__main__":
    main()
