"""Partition of one attention batch over the GPUs of one box and the gather of the results.

Every (fragment, head) pair is independent (spans never cross fragments), so ranks take contiguous blocks of
units (unit = fragment * heads + head) and no data crosses GPUs on the way in.  The partition itself is the
library's (tsa_shard_range / tsa_shard_rects, C ABI); this module binds it and carries the one collective of the
path, the all-gather of the output blocks, through `torch.distributed` (NCCL on GPUs, gloo in the CPU tests) or, fused into the attention kernel, as stores into the
other ranks' buffers (FusedGather: symmetric memory + tsa_att_fwd_to).
One process per GPU, as the reference runs one context and host thread per device
(code/gpt/compute/gpt_cuda.cu:1478-1738).
"""
import ctypes

import torch
import torch.distributed as dist

from . import abi


class Rect(ctypes.Structure):
    """tsa_shard_rect: fragments [frag_begin, frag_end) x heads [head_begin, head_end)"""
    _fields_ = [("frag_begin", ctypes.c_int), ("frag_end", ctypes.c_int), ("head_begin", ctypes.c_int), ("head_end", ctypes.c_int)]

    def as_tuple(self):
        return (self.frag_begin, self.frag_end, self.head_begin, self.head_end)


def split_range(n_units, world, rank):
    """Contiguous, balanced [begin, end) block of n_units for this rank (earlier ranks take the remainder)."""
    b, e = ctypes.c_int(0), ctypes.c_int(0)
    abi.check(abi.lib().tsa_shard_range(n_units, world, rank, ctypes.byref(b), ctypes.byref(e)))
    return b.value, e.value


def unit_rects(begin, end, heads):
    """The unit range [begin, end) as at most three (frag_begin, frag_end, head_begin, head_end) rectangles."""
    rects = (Rect * 3)()
    n = abi.lib().tsa_shard_rects(begin, end, heads, ctypes.cast(rects, ctypes.c_void_p))
    if n < 0:
        abi.check(-n)
    return [rects[i].as_tuple() for i in range(n)]


def rank_rects(fragments, heads, world, rank):
    """Rectangles of the (fragment, head) units this rank computes."""
    b, e = split_range(fragments * heads, world, rank)
    return unit_rects(b, e, heads)


def head_shard(heads, world, rank):
    """Heads owned by this rank when a single fragment is sharded by heads."""
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


def gather_blocks(local_block, gathered, group=None, async_op=False):
    """All-gather of equally shaped compact output blocks: local_block [rows][cols] (contiguous) from every rank into
    gathered [world][rows][cols].  Returns the work handle when async_op."""
    return dist.all_gather_into_tensor(gathered.view(-1), local_block.view(-1), group=group, async_op=async_op)


def unit_checksums(block, n_frag, seq, n_heads, head_dim):
    """Order-independent integer checksum of every (fragment, head) unit of a [n_frag * seq][n_heads * head_dim] block of
    16-bit values: the sum of the bit patterns (as signed 16-bit integers) of the unit's elements.  int64 [n_frag][n_heads]."""
    bits = block.view(torch.int16).to(torch.int64)
    return bits.view(n_frag, seq, n_heads, head_dim).sum(dim=(1, 3))


class FusedGather:
    """Buffers for the all-gather that the forward kernel does itself (tsa_att_fwd_to): every rank holds the whole output,
    [slices][world][rows][cols], in symmetric memory, i.e. mapped into every process of the box, and a rank's attention
    kernel stores its block of slice s into `local(s)` and, through `peers(s)`, into the same place of every other rank's
    buffer (plain peer stores over NVLink; no collective, no multicast).  `barrier()` is the stream-ordered cross-rank
    barrier that ends a step: past it every block of every buffer is complete."""

    def __init__(self, n_slices, rows, cols, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.whole = symm.empty((n_slices, self.world, rows, cols), dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.whole, group)
        self._ptrs = [int(x) for x in self.handle.buffer_ptrs]
        self._block = rows * cols * self.whole.element_size()
        self._stride = cols * self.whole.element_size()

    def gathered(self, s):
        """[world][rows][cols]: slice s of every rank's block, as this rank holds it"""
        return self.whole[s]

    def local(self, s):
        return self.whole[s][self.rank]

    def peers(self, s):
        """(address, row stride in bytes) of this rank's block of slice s inside every OTHER rank's buffer"""
        off = (s * self.world + self.rank) * self._block
        return [(self._ptrs[q] + off, self._stride) for q in range(self.world) if q != self.rank]

    def barrier(self):
        self.handle.barrier()

    def scatter(self, s, ctas=0, stream=None):
        """Copies this rank's block of slice s into every other rank's buffer with the library's own copy kernel
        (tsa_peer_scatter) on `stream` (default: the current one)."""
        from . import ops
        src = self.local(s)
        peers = self.peers(s)
        dsts = (ops.Ptr2D * len(peers))()
        for i, (ptr, stride) in enumerate(peers):
            dsts[i] = ops.Ptr2D(ptr, stride, src.shape[1], src.shape[0])
        st = stream if stream is not None else torch.cuda.current_stream()
        abi.check(abi.lib().tsa_peer_scatter(ops.p2d(src), dsts, len(peers), src.shape[0], src.shape[1] * src.element_size(), ctas,
                                             ctypes.c_void_p(st.cuda_stream)))
