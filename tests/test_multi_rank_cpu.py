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
