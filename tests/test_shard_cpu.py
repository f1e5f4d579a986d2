"""Row sharding across ranks, on CPU with the gloo backend (world size 2):
shards of the packed matrix, run through the oracle on each rank and
all-gathered, reproduce the unsharded oracle exactly."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import if_i_could_turn_back_time_b200 as jq
        from if_i_could_turn_back_time_b200 import dist as jd
        from oracle import formats
        g = torch.Generator("cpu").manual_seed(7)
        W = torch.randn(64, 256, generator=g) * 0.02
        x = torch.randn(3, 256, generator=g)
        for spec in (jq.QuantSpec("gf4", 128, 128), jq.QuantSpec("e2m1", 32, 0)):
            pw = jq.pack_weight(W, spec)                      # every rank packs the same full matrix
            mine = jd.shard_rows(pw, rank, world)
            assert mine.N == 32 and mine.qweight.shape[0] == 32

            def dq(p):
                codes = formats.unpack_nibbles(p.qweight.numpy(), p.K)
                if spec.fmt == "gf4":
                    return formats.dequant_gf4(codes, p.codebook.numpy(), p.scales.numpy(), 128)
                return formats.dequant_e2m1(codes, p.scales.numpy(), 32)

            y_local = torch.from_numpy(formats.linear_ref(x.numpy(), dq(mine), None, spec.had_block))
            y = jd.gather_rows(y_local)
            y_full = formats.linear_ref(x.numpy(), dq(pw), None, spec.had_block)
            assert y.shape == (3, 64)
            assert np.array_equal(y.numpy(), y_full), "sharded + gathered differs from unsharded"
            # packing a shard directly equals slicing the packed matrix (formats are per row)
            lo, hi = jd.shard_bounds(64, rank, world)
            direct = jq.pack_weight(W[lo:hi], spec)
            assert torch.equal(direct.qweight, mine.qweight)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_row_shard_all_gather_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


def test_shard_bounds_reject_uneven_split():
    from if_i_could_turn_back_time_b200 import dist as jd
    assert jd.shard_bounds(1024, 3, 8) == (384, 512)
    with pytest.raises(ValueError):
        jd.shard_bounds(1000, 0, 3)
