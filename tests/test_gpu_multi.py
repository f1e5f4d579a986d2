"""Row-sharded execution on 2 GPUs (one process per GPU, NCCL): the all-gather
fused into the GEMV epilogue (peer stores into symmetric memory) and the plain
NCCL all-gather must both reproduce the unsharded result bit for bit.  Skipped
on a box with fewer than two GPUs.  NVLS is switched off for these child
processes and the kernels use plain peer stores only."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import if_i_could_turn_back_time_b200 as jq
        from if_i_could_turn_back_time_b200 import ops, dist as jd
        spec = jq.QuantSpec("gf4", 128, 128)
        shapes = [(512, 1024), (256, 2048), (1024, 256)]
        g = torch.Generator("cpu").manual_seed(3)
        Ws = [torch.randn(n, k, generator=g) * 0.02 for n, k in shapes]
        xs = [torch.randn(2, k, generator=g).bfloat16() for _, k in shapes]
        full = [jq.pack_weight(W, spec) for W in Ws]
        ref = [ops.linear(x.to(dev), pw.to(dev)) for x, pw in zip(xs, full)]
        shards = [jd.shard_rows(pw, rank, world).to(dev) for pw in full]
        # (1) fused exchange
        grp = ops.GroupedGemv(shards, 2, torch.bfloat16, full_rows=[pw.N for pw in full],
                              row_offsets=[jd.shard_bounds(pw.N, rank, world)[0] for pw in full],
                              group=dist.group.WORLD)
        assert grp.fused_exchange
        for step in range(3):   # repeated steps reuse the same symmetric arena
            for gx, x in zip(grp.xs, xs):
                gx.copy_(x * (step + 1))
            grp.barrier()       # nobody overwrites an arena a peer may still be reading
            grp.run()
            grp.barrier()
            torch.cuda.synchronize()
            for y, x, pw in zip(grp.ys, xs, full):
                want = ops.linear((x * (step + 1)).to(dev), pw.to(dev))
                assert torch.equal(y, want), f"rank {rank} step {step}: fused exchange differs"
        # (2) NCCL all-gather of the local slices
        for x, pw, sh, r in zip(xs, full, shards, ref):
            y = jd.gather_rows(ops.linear(x.to(dev), sh))
            assert torch.equal(y, r), f"rank {rank}: nccl gather differs"
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_row_shard_exchange_two_gpus():
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, 29600 + os.getpid() % 300, ret), nprocs=2, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}
