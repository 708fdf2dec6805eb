"""Host-side pieces of the data-parallel step driver (one process per GPU).

The frozen quantized base and the adapters are replicated; each rank processes its own sequences; after the
backward pass the flat fp32 LoRA-gradient buffer is summed across ranks and scaled by 1/world, which reproduces
the reference's gradient-accumulation averaging (src/Glacier.Tune/Trainer/LoraTrainer.cs:217-220) with ranks in
the place of micro-batches.  On GPUs the sum is the library's NCCL all-reduce (gt_dp_allreduce); the functions
here are the parts that need no GPU: the layout of the flat buffer and the rendezvous of the NCCL id.
"""
from __future__ import annotations

from typing import Iterable

PROJ_ORDER = ("q", "k", "v", "o", "gate", "up", "down")


def flat_grad_layout(proj_shapes: Iterable[tuple[str, int, int]], rank: int, layers: int = 1):
    """Offsets of (dA [in, r], dB [r, out]) per layer and projection inside one flat buffer.

    Order follows the reference's parameter list: layer, then q, k, v, o, gate, up, down, then A before B
    (src/Glacier.Tune/Model/TransformerBlock.cs:167-174).  proj_shapes yields (name, out_features, in_features).
    Returns (entries, total) with entries[(layer, name)] = (offset_dA, size_dA, offset_dB, size_dB).
    """
    shapes = list(proj_shapes)
    entries, off = {}, 0
    for layer in range(layers):
        for name, out_f, in_f in shapes:
            na, nb = in_f * rank, rank * out_f
            entries[(layer, name)] = (off, na, off + na, nb)
            off += na + nb
    return entries, off


BACKWARD_GROUPS = (("down",), ("gate", "up"), ("o",), ("q", "k", "v"))      # order in which a block's backward finishes them


def group_buckets(entries, layer: int = 0, groups=BACKWARD_GROUPS):
    """(offset, size) of each projection group's gradients inside the flat buffer, in backward order: the slices the
    overlapped exchange (gt_dp_allreduce_begin) sends as soon as the group's backward has produced them.  The members of
    a group are adjacent in the reference's parameter order, so every bucket is one contiguous slice."""
    out = []
    for g in groups:
        a0 = entries[(layer, g[0])][0]
        ob, nb = entries[(layer, g[-1])][2], entries[(layer, g[-1])][3]
        for name in g[1:]:      # adjacency check
            prev = g[g.index(name) - 1]
            assert entries[(layer, name)][0] == entries[(layer, prev)][2] + entries[(layer, prev)][3], "group members must be adjacent"
        out.append((a0, ob + nb - a0))
    return out


def layer_buckets(entries, layers: int, proj_order=PROJ_ORDER):
    """(offset, size) of each layer's gradients inside the flat buffer, LAST layer first: the slices the training-step
    driver (gt_model_forward_backward) all-reduces as soon as a block's backward is queued, beside the backward of
    the blocks below it.  A layer's seven adapters are adjacent in the reference's parameter order."""
    out = []
    for layer in range(layers - 1, -1, -1):
        first, last = entries[(layer, proj_order[0])], entries[(layer, proj_order[-1])]
        out.append((first[0], last[2] + last[3] - first[0]))
    return out


def share_unique_id(make_id, dist_module, src: int = 0) -> bytes:
    """Rank `src` creates the communicator id; every rank returns the same bytes (torch.distributed rendezvous)."""
    box = [make_id() if dist_module.get_rank() == src else None]
    dist_module.broadcast_object_list(box, src=src)
    return box[0]


def average_gradients_reference(flat, dist_module) -> None:
    """The same reduction with torch.distributed (gloo on CPU): sum over ranks, then 1/world.  Used by the CPU tests
    of the driver logic; the GPU path calls gt_dp_allreduce instead."""
    dist_module.all_reduce(flat)
    flat.mul_(1.0 / dist_module.get_world_size())


def average_gradients_bucketed(flat, buckets, dist_module) -> None:
    """The bucketed form of the same reduction: one all-reduce per (offset, size) slice in the given order, the order in
    which a backward pass finishes them.  On GPUs each slice is a gt_dp_allreduce_begin call; the result is the same as
    one all-reduce over the whole buffer."""
    inv = 1.0 / dist_module.get_world_size()
    for off, size in buckets:
        part = flat[off: off + size]
        dist_module.all_reduce(part)
        part.mul_(inv)
