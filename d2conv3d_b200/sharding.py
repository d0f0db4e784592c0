"""Multi-GPU plumbing of the path: one process per GPU, clips (the batch dimension) sharded across
ranks, weights replicated, and a single collective -- the sum of grad_weight / grad_bias -- for
training-style runs.  Forward, grad_input, grad_offset and grad_mask depend only on a rank's own
clips (reference csrc/ops/dconv3d_gpu.cu:147,158-178 offsets every pointer by the clip index), so the
data path needs no exchange; the reference's DDP wrapper (trainer.py:111) all-reduces parameter
gradients the same way.

Works with any torch.distributed backend: NCCL on GPUs, gloo in the CPU tests.
"""
import torch
import torch.distributed as dist


def clip_range(n_clips, rank, world_size):
    """Contiguous slice [begin, end) of the batch owned by `rank`; sizes differ by at most one."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(n_clips, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_clips(tensors, rank=None, world_size=None):
    """Slices every tensor (or None) of `tensors` along dim 0 to this rank's clips."""
    rank = dist.get_rank() if rank is None else rank
    world_size = dist.get_world_size() if world_size is None else world_size
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        b, e = clip_range(t.shape[0], rank, world_size)
        out.append(t[b:e])
    return out


def all_reduce_param_grads(grads, group=None, async_op=False):
    """Sums parameter gradients (grad_weight, grad_bias; None entries skipped) over all ranks, as ONE flat
    bucket so that small gradients cost a single collective.

    Always returns `(work, finish)`: `work` is the collective's handle (None when nothing had to be launched or
    the call was synchronous) and `finish()` waits for it (if needed) and copies the reduced values back into
    the gradient tensors.  With async_op=False `finish` has already run and is a no-op to call again."""
    live = [g for g in grads if g is not None]
    if not live or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None, (lambda: None)
    flat = live[0].reshape(-1) if (len(live) == 1 and live[0].is_contiguous()) else \
        torch.cat([g.reshape(-1) for g in live])
    in_place = len(live) == 1 and flat.data_ptr() == live[0].data_ptr()
    work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
    state = {"done": False}

    def finish():
        if state["done"]:
            return
        if work is not None:
            work.wait()
        if not in_place:
            off = 0
            for g in live:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n
        state["done"] = True

    if not async_op:
        finish()
        return None, finish
    return work, finish


def all_reduce_param_grads_overlapped(grads, ready_event, side_stream, group=None):
    """The DDP-style overlap for this layer: `side_stream` waits for `ready_event` (the event the library records
    when grad_weight / grad_bias are final, `dconv_native._ops.params_ready_event()`), the flat-bucket all-reduce
    of all_reduce_param_grads is issued from there, and the stream that was current at the call -- on which the
    rest of the backward is still running -- is NOT made to wait.  Returns `finish`: call it on the compute stream
    before the gradients are used (it makes the current stream wait for the collective and unpacks the bucket).
    Single rank or no process group: returns a no-op."""
    live = [g for g in grads if g is not None]
    if not live or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return lambda: None
    if ready_event is not None:
        side_stream.wait_event(ready_event)
    else:
        side_stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side_stream):
        work, finish_side = all_reduce_param_grads(live, group=group, async_op=True)
        for g in live:
            g.record_stream(side_stream)

    def finish():
        with torch.cuda.stream(side_stream):
            finish_side()
        torch.cuda.current_stream().wait_stream(side_stream)

    return finish


def broadcast_params(params, src=0, group=None):
    """Replicates weights / bias from `src` at start-up."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for p in params:
        if p is not None:
            dist.broadcast(p.data if hasattr(p, "data") else p, src=src, group=group)
