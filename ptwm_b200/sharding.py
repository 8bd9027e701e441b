"""Splitting one container across the GPUs of a box.

Tensors are independent, so a rank decodes a contiguous run of records (in
file order) and needs only that byte range of the file on its GPU.  There is
no exchange step on that path.

When every rank needs the whole model (data-parallel replicas), the bytes that
cross PCIe are still split: each rank copies only its own span of the
*compressed* container to its GPU, the spans are exchanged over NVLink with
NCCL (`all_gather_compressed`: one broadcast per owner, straight into place in
every rank's buffer), and every rank then decodes the whole container from its
own memory (`decode_replica`).  The decode kernels only ever read local memory;
no peer pointer reaches a kernel.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def contiguous_shards(costs: Sequence[int], world: int) -> list[range]:
    """Partition items 0..n-1 into `world` contiguous ranges whose summed
    cost is as even as a greedy left-to-right cut makes it: rank r ends at
    the first item where the running cost reaches (r+1)/world of the total."""
    n = len(costs)
    total = sum(costs)
    bounds = [0]
    run = 0
    i = 0
    for r in range(1, world):
        target = total * r / world
        while i < n and run + costs[i] / 2 <= target:
            run += costs[i]
            i += 1
        bounds.append(i)
    bounds.append(n)
    return [range(bounds[r], bounds[r + 1]) for r in range(world)]


def shard_for_rank(infos: Sequence[dict], rank: int, world: int) -> list[int]:
    """Indices of the tensors rank `rank` of `world` decodes.  Cost of a
    tensor = compressed bytes read + decoded bytes written."""
    costs = [int(t["compressed"]) + int(t["orig_size"]) for t in infos]
    return list(contiguous_shards(costs, world)[rank])


def replica_spans(infos: Sequence[dict], world: int) -> list[tuple[int, int]]:
    """File byte range [lo, hi) each rank brings to the exchange: the ranges are
    disjoint, in rank order, and tile the range from the first payload byte of
    the first supported tensor to the last payload byte of the last one (bytes
    between two tensors' payloads, record headers, travel with the earlier
    rank).  Cut like `shard_for_rank`, by compressed bytes only: what a rank
    copies and sends is compressed bytes."""
    live = [i for i, t in enumerate(infos) if t.get("supported", True) and t["end_byte"] > t["first_byte"]]
    if not live:
        return [(0, 0)] * world
    parts = contiguous_shards([int(infos[i]["compressed"]) for i in live], world)
    lo_all, hi_all = min(infos[i]["first_byte"] for i in live), max(infos[i]["end_byte"] for i in live)
    starts = []
    for r in range(world):
        starts.append(min(infos[live[j]]["first_byte"] for j in parts[r]) if len(parts[r]) else None)
    spans, nxt = [], hi_all
    for r in reversed(range(world)):  # a rank's range ends where the next non-empty one starts
        if starts[r] is None:
            spans.append((nxt, nxt))
        else:
            spans.append((starts[r], nxt))
            nxt = starts[r]
    spans.reverse()
    first = next(r for r in range(world) if starts[r] is not None)
    spans[first] = (lo_all, spans[first][1])
    return spans


REPLICA_SLICES = 4


def span_slices(a: int, b: int, pieces: int = REPLICA_SLICES, align: int = 1 << 20) -> list[tuple[int, int]]:
    """[a, b) cut into at most `pieces` contiguous parts of equal length (a multiple of `align`, the last one shorter), none empty."""
    if b <= a:
        return []
    step = -(-(-(-(b - a) // pieces)) // align) * align
    return [(x, min(b, x + step)) for x in range(a, b, step)]


def all_gather_compressed(host_blob: torch.Tensor, infos: Sequence[dict], group=None, device=None):
    """Every rank ends up with file bytes [lo, hi) of the container in its own
    memory: it copies its own span from `host_blob` (the container in host
    memory, pinned for an asynchronous copy) and receives the other spans from
    their owners, one NCCL broadcast per owner, each landing at its final offset.
    Returns (buffer, lo, bytes received from peers).  `device=None` keeps
    everything in host memory (gloo; used to test the bookkeeping without GPUs)."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    spans = replica_spans(infos, world)
    lo, hi = spans[0][0], spans[-1][1]
    dev = torch.device("cpu") if device is None else torch.device("cuda", int(device))
    buf = torch.empty(max(hi - lo, 1), dtype=torch.uint8, device=dev)
    a, b = spans[rank]
    received = sum(rb - ra for r, (ra, rb) in enumerate(spans) if r != rank) if world > 1 else 0

    def src_of(r):
        return dist.get_global_rank(group, r) if group is not None else r

    if device is None or world == 1:
        if b > a:
            buf[a - lo:b - lo].copy_(host_blob[a:b], non_blocking=True)
        if world > 1:
            for r, (ra, rb) in enumerate(spans):
                if rb > ra:
                    dist.broadcast(buf[ra - lo:rb - lo], src=src_of(r), group=group)
        return buf, lo, received
    # On GPUs a span travels in slices: slice k of every span is broadcast while slice k + 1 is still crossing PCIe,
    # so NVLink works beside the host copies instead of after them.  The cuts are a function of the span alone:
    # every rank makes the same calls in the same order.
    copier = torch.cuda.Stream(dev)
    buf.record_stream(copier)
    landed = []
    with torch.cuda.stream(copier):
        copier.wait_stream(torch.cuda.current_stream(dev))
        for sa, sb in span_slices(a, b):
            buf[sa - lo:sb - lo].copy_(host_blob[sa:sb], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copier)
            landed.append(ev)
    cuts = [span_slices(ra, rb) for ra, rb in spans]
    works = []
    for k in range(max((len(c) for c in cuts), default=0)):
        for r in range(world):
            if k < len(cuts[r]):
                sa, sb = cuts[r][k]
                if r == rank:
                    torch.cuda.current_stream(dev).wait_event(landed[k])  # the collective starts after what the current stream waits for
                works.append(dist.broadcast(buf[sa - lo:sb - lo], src=src_of(r), group=group, async_op=True))
    for w in works:
        w.wait()
    return buf, lo, received


def decode_replica(handle, group=None, names: Optional[Sequence[str]] = None):
    """The whole model on every rank of `group`: PCIe carries 1 / world of the
    compressed container per rank, NVLink the rest, then one local decode pass.
    `handle` is a ContainerHandle over the container in (pinned) host memory,
    opened whole on every rank.  Returns ([(name, tensor)], bytes received over NVLink)."""
    infos = handle.tensor_infos()
    buf, lo, received = all_gather_compressed(handle._host, infos, group, handle.device)
    indices = None if names is None else [handle._idx(n) for n in names]
    plan = handle.plan(indices)
    plo, phi = plan.blob_span
    dev = torch.device("cuda", handle.device)
    out = torch.empty(plan.out_bytes, dtype=torch.uint8, device=dev)
    scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device=dev) if plan.scratch_bytes else None
    if phi > plo and (plo < lo or phi > lo + buf.numel()):
        raise RuntimeError("internal: the gathered range does not cover the plan")
    plan.run(buf[plo - lo:phi - lo] if phi > plo else buf[:0], out, scratch, blob_first=plo, flags=handle._flags())
    return [(infos[i]["name"], v) for i, v in zip(plan.indices, plan.views(out))], received
