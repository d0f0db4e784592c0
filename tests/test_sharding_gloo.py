"""World-size-2 CPU (gloo) test of the multi-GPU plumbing: clip sharding + the grad_weight / grad_bias
all-reduce.  The per-rank compute is the CPU oracle here (test infrastructure standing in for the GPU
kernels); what is under test is that sharded results + the one collective reproduce the full-batch
result: outputs and per-clip gradients concatenate, parameter gradients sum."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from d2conv3d_b200 import sharding
from tests._util import make_problem


def test_clip_range_partitions_the_batch():
    for n in (1, 2, 5, 8, 32):
        for w in (1, 2, 3, 4, 8):
            covered = []
            for r in range(w):
                b, e = sharding.clip_range(n, r, w)
                covered += list(range(b, e))
            assert covered == list(range(n))
            sizes = [sharding.clip_range(n, r, w)[1] - sharding.clip_range(n, r, w)[0] for r in range(w)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.clip_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc
    p = make_problem(900, 5, 4, 6, (3, 5, 5), padding=1, G=2, dtype=np.float64)   # 5 clips over 2 ranks: 3 + 2
    kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=2)
    w = torch.from_numpy(p["weight"]).clone()
    bias = torch.from_numpy(p["bias"]).clone()
    if rank != 0:
        w.zero_(); bias.zero_()
    sharding.broadcast_params([w, bias])                      # weights replicated from rank 0
    x, off, m, gy = sharding.shard_clips([torch.from_numpy(p[k]) for k in ("x", "geo", "mask", "gy")])
    y = orc.deform_conv3d_fwd(x.numpy(), off.numpy(), m.numpy(), w.numpy(), bias.numpy(), **kw)
    gx, goff, gm, gw, gb = orc.deform_conv3d_bwd(gy.numpy(), x.numpy(), off.numpy(), m.numpy(), w.numpy(), True, **kw)
    gw_t, gb_t = torch.from_numpy(gw), torch.from_numpy(gb)
    work, finish = sharding.all_reduce_param_grads([gw_t, None, gb_t])       # the only collective
    assert work is None
    finish()                                                  # synchronous call: already done, a no-op
    # the asynchronous form returns the same (work, finish) shape; values land when finish() returns
    probe = [torch.full((3,), float(rank + 1)), torch.full((2, 2), 10.0 * (rank + 1))]
    work, finish = sharding.all_reduce_param_grads(probe, async_op=True)
    assert work is not None
    finish()
    assert torch.all(probe[0] == 3.0) and torch.all(probe[1] == 30.0)
    single = [torch.full((4,), float(rank + 1))]
    work, finish = sharding.all_reduce_param_grads(single, async_op=True)
    finish()
    assert torch.all(single[0] == 3.0)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), y=y, gx=gx, goff=goff, gm=gm, gw=gw_t.numpy(), gb=gb_t.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_full_batch(tmp_path):
    from oracle import oracle as orc
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    p = make_problem(900, 5, 4, 6, (3, 5, 5), padding=1, G=2, dtype=np.float64)
    kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=2)
    y = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    gx, goff, gm, gw, gb = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, **kw)
    parts = [np.load(os.path.join(tmp_path, f"rank{r}.npz")) for r in range(world)]
    assert np.array_equal(np.concatenate([q["y"] for q in parts]), y)
    assert np.array_equal(np.concatenate([q["gx"] for q in parts]), gx)
    assert np.array_equal(np.concatenate([q["goff"] for q in parts]), goff)
    assert np.array_equal(np.concatenate([q["gm"] for q in parts]), gm)
    for q in parts:                                           # every rank holds the summed parameter gradients
        assert np.allclose(q["gw"], gw, rtol=1e-12, atol=1e-12)
        assert np.allclose(q["gb"], gb, rtol=1e-12, atol=1e-12)
