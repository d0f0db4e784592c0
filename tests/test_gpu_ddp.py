"""Data-parallel training step through real autograd on two GPUs: a modulated deformable layer wrapped in
torch's DistributedDataParallel (NCCL), clips sharded over the ranks with d2conv3d_b200.sharding, one forward +
backward per rank.  DDP's all-reduce of the parameter gradients is the only collective, as in the reference's
trainer (trainer.py:97-111); the averaged gradients must equal the single-GPU full-batch gradients divided by
the world size, and the per-clip input gradients must equal the full-batch ones.  Skipped with fewer than two
GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

REL = 1e-4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_layer(seed):
    from d2conv3d_b200.dconv_native import modules
    torch.backends.cudnn.allow_tf32 = False          # the predictor conv is cuDNN: keep it fp32 on both sides
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(seed)
    layer = modules.MDConv3d(64, 64, 3, padding=1, offset_groups=1)
    torch.nn.init.normal_(layer.deform_params.weight, std=0.05)      # non-trivial offsets and masks
    return layer


def _inputs(seed, clips):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((clips, 64, 3, 8, 10), generator=g)
    gy = torch.randn((clips, 64, 3, 8, 10), generator=g)
    return x, gy


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from d2conv3d_b200 import _lib, sharding
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    layer = _make_layer(77).to(dev)
    ddp = DDP(layer, device_ids=[rank])
    x, gy = _inputs(78, 4)
    x, gy = sharding.shard_clips([x, gy])
    x = x.to(dev).requires_grad_()
    y = ddp(x)
    y.backward(gy.to(dev))
    torch.cuda.synchronize()
    _lib.device_status()
    torch.save({"gx": x.grad.cpu(), "y": y.detach().cpu(),
                "grads": {n: p.grad.cpu() for n, p in layer.named_parameters()}},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ddp_step_matches_single_gpu_full_batch(tmp_path):
    import torch.multiprocessing as mp

    from d2conv3d_b200 import _lib
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    # single GPU, full batch
    dev = torch.device("cuda", 0)
    layer = _make_layer(77).to(dev)
    x, gy = _inputs(78, 4)
    x = x.to(dev).requires_grad_()
    y = layer(x)
    y.backward(gy.to(dev))
    _lib.device_status()
    outs = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]

    def rel(a, b):
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))

    assert rel(torch.cat([o["y"] for o in outs]), y.detach().cpu()) <= REL
    assert rel(torch.cat([o["gx"] for o in outs]), x.grad.cpu()) <= REL
    for name, p in layer.named_parameters():
        want = p.grad.cpu() / world                      # DDP averages over ranks
        for o in outs:                                   # and every rank holds the same averaged gradient
            assert rel(o["grads"][name], want) <= REL, name
