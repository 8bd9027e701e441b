"""World-size-2 check of the multi-GPU path's host logic on CPU (gloo): every
rank parses the same container, takes its contiguous run of records, builds
its plan and byte span; together the ranks cover every tensor once and their
spans stay inside the file.  No data-path collective exists, so the only
traffic here is the test's own gather of the results."""
import ctypes as C
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "oracle", "mixed_chunk4k_crc.ptwm")


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ptwm_b200 import _lib
    from ptwm_b200.sharding import shard_for_rank
    L = _lib.lib()
    blob = open(GOLD, "rb").read()
    buf = (C.c_char * len(blob)).from_buffer_copy(blob)
    h = C.c_void_p()
    assert L.ptwm_b200_open(C.addressof(buf), len(blob), C.byref(h)) == 0
    infos = []
    for i in range(L.ptwm_b200_tensor_count(h)):
        ti = _lib.TensorInfo()
        L.ptwm_b200_tensor_info_get(h, i, C.byref(ti))
        infos.append(dict(compressed=ti.compressed, orig_size=ti.orig_size, first_byte=ti.first_byte, end_byte=ti.end_byte))
    mine = shard_for_rank(infos, rank, world)
    arr = (C.c_uint32 * max(len(mine), 1))(*mine)
    p = C.c_void_p()
    assert L.ptwm_b200_plan_create(h, arr, len(mine), C.byref(p)) == 0
    lo, hi = C.c_uint64(), C.c_uint64()
    L.ptwm_b200_plan_blob_span(p, C.byref(lo), C.byref(hi))
    r, w, n = C.c_uint64(), C.c_uint64(), C.c_uint32()
    L.ptwm_b200_plan_stats(p, C.byref(r), C.byref(w), C.byref(n))
    result = dict(rank=rank, mine=mine, span=(lo.value, hi.value), written=w.value, expect=sum(infos[i]["orig_size"] for i in mine),
                  inside=min(infos[i]["first_byte"] for i in mine) <= lo.value and hi.value <= max(infos[i]["end_byte"] for i in mine),
                  n=len(infos), size=len(blob))
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        q.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_cover_the_container():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(i for r in res for i in r["mine"]) == list(range(res[0]["n"]))
    assert all(r["written"] == r["expect"] and r["inside"] and r["span"][1] <= r["size"] for r in res)
    assert res[0]["span"][1] <= res[1]["span"][0] + 1 or res[0]["span"][0] < res[1]["span"][0]  # contiguous runs: rank 0's bytes come first
    assert all(len(r["mine"]) > 0 for r in res)


# ---- replica mode: every rank ends up with the whole compressed range ----------------------------
def _gather_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ptwm_b200 import _lib
    from ptwm_b200.sharding import all_gather_compressed, replica_spans
    L = _lib.lib()
    blob = open(GOLD, "rb").read()
    buf = (C.c_char * len(blob)).from_buffer_copy(blob)
    h = C.c_void_p()
    assert L.ptwm_b200_open(C.addressof(buf), len(blob), C.byref(h)) == 0
    infos = []
    for i in range(L.ptwm_b200_tensor_count(h)):
        ti = _lib.TensorInfo()
        L.ptwm_b200_tensor_info_get(h, i, C.byref(ti))
        infos.append(dict(compressed=ti.compressed, orig_size=ti.orig_size, first_byte=ti.first_byte, end_byte=ti.end_byte, supported=bool(ti.supported)))
    host = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
    if rank == 1:  # a rank must not depend on bytes outside its own span being present in its host copy
        a, b = replica_spans(infos, world)[rank]
        mask = torch.ones_like(host, dtype=torch.bool)
        mask[a:b] = False
        host[mask] = 0xEE
    got, lo, received = all_gather_compressed(host, infos, None, None)
    spans = replica_spans(infos, world)
    ok = got.numpy().tobytes() == blob[lo:lo + got.numel()]
    result = dict(rank=rank, ok=ok, lo=lo, n=got.numel(), received=received, spans=spans)
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        q.put((gathered, [(t["first_byte"], t["end_byte"]) for t in infos if t["end_byte"] > t["first_byte"]]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_exchange_their_compressed_spans():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res, payloads = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r["ok"] for r in res)
    spans = res[0]["spans"]
    assert spans == res[1]["spans"] and spans[0][1] == spans[1][0] and spans[0][0] < spans[0][1] < spans[1][1]  # disjoint, in order, tiling
    assert spans[0][0] == min(a for a, _ in payloads) and spans[1][1] == max(b for _, b in payloads)
    assert res[0]["lo"] == spans[0][0] and res[0]["n"] == spans[1][1] - spans[0][0]
    assert res[0]["received"] == spans[1][1] - spans[1][0] and res[1]["received"] == spans[0][1] - spans[0][0]


def test_replica_spans_edge_cases():
    from ptwm_b200.sharding import replica_spans
    infos = [dict(compressed=10, first_byte=100, end_byte=110), dict(compressed=0, first_byte=0, end_byte=0, supported=False),
             dict(compressed=30, first_byte=120, end_byte=150)]
    assert replica_spans(infos, 1) == [(100, 150)]
    two = replica_spans(infos, 2)
    assert two[0][0] == 100 and two[-1][1] == 150 and two[0][1] == two[1][0]
    many = replica_spans(infos, 4)  # more ranks than tensors: the extra ranks bring nothing
    assert many[0][0] == 100 and many[-1][1] == 150 and all(a <= b for a, b in many) and all(many[i][1] == many[i + 1][0] for i in range(3))
    assert replica_spans([], 3) == [(0, 0)] * 3


def test_span_slices_tile_the_span():
    from ptwm_b200.sharding import REPLICA_SLICES, span_slices
    for a, b in [(0, 0), (5, 6), (100, 5_000_100), (123_456_789, 1_423_456_789), (0, 1 << 20), (7, (1 << 20) + 9), (3, 3 + 4 * (1 << 20) + 1)]:
        cuts = span_slices(a, b)
        assert len(cuts) <= REPLICA_SLICES
        if a == b:
            assert cuts == []
            continue
        assert cuts[0][0] == a and cuts[-1][1] == b and all(x[1] == y[0] for x, y in zip(cuts, cuts[1:])) and all(y > x for x, y in cuts)
