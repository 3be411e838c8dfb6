"""Partition of the attention work over the GPUs of one box and the gather of the results.

Every (fragment, head) pair is independent (spans never cross fragments), so ranks take contiguous blocks of
heads (or of fragments) and no data crosses GPUs on the way in.  The only collective is the all-gather of the
output column blocks.  One process per GPU; `torch.distributed` carries the collective (NCCL on GPUs, gloo in
the CPU tests).
"""
import torch
import torch.distributed as dist


def split_range(n_units, world, rank):
    """Contiguous, balanced [begin, end) block of n_units for this rank (earlier ranks take the remainder)."""
    base, rem = divmod(n_units, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def head_shard(heads, world, rank):
    """Heads owned by this rank when a layer is sharded by heads."""
    return split_range(heads, world, rank)


def gather_head_blocks(local_out, heads, head_dim, world, group=None):
    """All-gather of per-rank output column blocks [len][heads_local * head_dim] into [len][heads * head_dim].
    Ranks may own different numbers of heads; blocks are padded to the largest for the collective."""
    if world == 1:
        return local_out
    length = local_out.shape[0]
    counts = [split_range(heads, world, r)[1] - split_range(heads, world, r)[0] for r in range(world)]
    width = max(counts) * head_dim
    send = local_out
    if local_out.shape[1] != width:
        send = torch.zeros((length, width), dtype=local_out.dtype, device=local_out.device)
        send[:, :local_out.shape[1]] = local_out
    recv = torch.empty((world, length, width), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(recv.view(-1), send.contiguous().view(-1), group=group)
    parts = [recv[r, :, :counts[r] * head_dim] for r in range(world)]
    return torch.cat(parts, dim=1)
