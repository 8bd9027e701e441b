"""Host-side logic of the CUDA library, without a GPU: the C ABI loads and
exports what include/ptwm_b200.h declares, the container parser agrees with
the oracle's, plans are sized sensibly and malformed input is refused."""
import ctypes as C
import json
import os
import re
import zlib

import numpy as np
import pytest

import oracle
import ptwm_b200
from ptwm_b200 import _lib
from ptwm_b200.sharding import contiguous_shards, shard_for_rank

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def L():
    ptwm_b200.build()
    return _lib.lib()


def _open(L, blob):
    buf = (C.c_char * len(blob)).from_buffer_copy(blob)
    h = C.c_void_p()
    rc = L.ptwm_b200_open(C.addressof(buf), len(blob), C.byref(h))
    return rc, h


def _infos(L, h):
    out = []
    for i in range(L.ptwm_b200_tensor_count(h)):
        ti = _lib.TensorInfo()
        assert L.ptwm_b200_tensor_info_get(h, i, C.byref(ti)) == 0
        out.append(ti)
    return out


def test_every_declared_symbol_is_exported(L):
    header = open(os.path.join(ROOT, "include", "ptwm_b200.h")).read()
    declared = set(re.findall(r"\b(ptwm_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(L, name), name


def test_crc_fold_matches_zlib(L):
    rng = np.random.default_rng(0)
    for n in [0, 1, 5, 2047, 2048, 2049, 10000, 300001]:
        b = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        for run in [1, 7, 2048, 1 << 20]:
            assert L.ptwm_b200_crc32_by_runs(b, n, run) == zlib.crc32(b)


def test_parser_agrees_with_oracle_on_goldens(L):
    man = json.load(open(os.path.join(GOLD, "oracle", "manifest.json")))
    for name in man:
        if name == "frames":
            continue
        blob = open(os.path.join(GOLD, "oracle", name + ".ptwm"), "rb").read()
        rc, h = _open(L, blob)
        assert rc == 0, _lib.last_error()
        oc = oracle.Container(blob)
        infos = _infos(L, h)
        assert [t.name.decode() for t in infos] == oc.names
        for ti, ot in zip(infos, oc.tensors):
            assert ti.supported and ti.orig_size == ot["orig_size"] and ti.dtype_code == ot["dtype_code"] and ti.kind == ot["kind"]
            assert list(ti.shape)[:ti.ndim] == ot["shape"] and bool(ti.has_hash) == ot["has_hash"]
            assert ti.compressed == sum(p["payload_len"] for p in ot["planes"])
        p = C.c_void_p()
        assert L.ptwm_b200_plan_create(h, None, 0, C.byref(p)) == 0, _lib.last_error()
        assert L.ptwm_b200_plan_out_bytes(p) >= sum(t["orig_size"] for t in oc.tensors)
        r, w, n = C.c_uint64(), C.c_uint64(), C.c_uint32()
        L.ptwm_b200_plan_stats(p, C.byref(r), C.byref(w), C.byref(n))
        assert w.value == sum(t["orig_size"] for t in oc.tensors) and 0 < r.value <= len(blob) and n.value >= 1
        lo, hi = C.c_uint64(), C.c_uint64()
        L.ptwm_b200_plan_blob_span(p, C.byref(lo), C.byref(hi))
        assert 0 < lo.value < hi.value <= len(blob)
        L.ptwm_b200_plan_destroy(p)
        L.ptwm_b200_close(h)


def test_reference_fixtures_open(L):
    blob = open(os.path.join(GOLD, "reference", "ptwc_bound_source"), "rb").read()
    rc, h = _open(L, blob)
    assert rc == 0
    infos = _infos(L, h)
    assert [t.name for t in infos] == [b"t1", b"t2", b"t3", b"t4"] and all(t.supported and t.kind == 2 and t.has_hash and t.has_crc for t in infos)
    L.ptwm_b200_close(h)
    # zstd planes and a delta-coded tensor: opens, tensors flagged as outside the hot path, planning refuses
    blob = open(os.path.join(GOLD, "reference", "ptwc_trimmed"), "rb").read()
    rc, h = _open(L, blob)
    assert rc == 0
    infos = _infos(L, h)
    assert len(infos) == 6 and not any(t.supported for t in infos)
    p = C.c_void_p()
    assert L.ptwm_b200_plan_create(h, None, 0, C.byref(p)) == -5  # Unsupported (native.rs:634-657)
    L.ptwm_b200_close(h)


def test_frames_open(L):
    for f in sorted(os.listdir(os.path.join(GOLD, "reference", "compact_decode"))):
        blob = b"\x89PTWS" + open(os.path.join(GOLD, "reference", "compact_decode", f), "rb").read()
        rc, h = _open(L, blob)
        assert rc == 0, (f, _lib.last_error())
        infos = _infos(L, h)
        assert len(infos) == 1 and infos[0].name == b"_"
        L.ptwm_b200_close(h)
        rc, h = _open(L, blob + b"\x00")  # a frame is self-delimiting
        if infos[0].supported:
            assert rc < 0


def test_every_byte_mutation_is_survived(L):
    # tests/ptwc.rs:130 of the reference: mutate each byte, the reader must answer (error or success), never crash
    blob = bytearray(open(os.path.join(GOLD, "reference", "ptwc_bound_source"), "rb").read())
    rejected = 0
    for i in range(len(blob)):
        m = bytearray(blob)
        m[i] ^= 0x5A
        rc, h = _open(L, bytes(m))
        if rc < 0:
            rejected += 1
        else:
            L.ptwm_b200_close(h)
    assert rejected > len(blob) // 4
    for cut in range(0, len(blob), 7):
        rc, h = _open(L, bytes(blob[:cut]))
        assert rc < 0


def test_legacy_fixtures_open(L):
    """The legacy \\x89PTWM layout: records in write order, shape metadata from the CBOR map, Zstd planes and the
    delta-coded tensor flagged as outside the hot path, the Order1ScaleAC and tANS tensors plannable."""
    for fixture in ("legacy_v1_1_0", "legacy_v1_0_0", "legacy_v1_0_0_native"):
        blob = open(os.path.join(GOLD, "reference", fixture + ".ptwm"), "rb").read()
        rc, h = _open(L, blob)
        assert rc == 0, fixture
        infos = _infos(L, h)
        assert [t.name.decode() for t in infos] == ["model.layers.0.q.weight", "model.layers.0.k.weight", "model.norm.weight", "model.layers.0.mlp.fp8.weight",
                                                    "model.embed.int8", "model.layers.0.q.scale", "model.layers.0.k.scale", "model.layers.1.q.weight",
                                                    "model.layers.2.chunked.weight"]
        ok = {t.name.decode(): t for t in infos if t.supported}
        want = {"model.layers.2.chunked.weight"} | ({"model.layers.0.q.scale", "model.layers.0.k.scale"} if "native" not in fixture else set())
        assert set(ok) == want, fixture
        t = ok["model.layers.2.chunked.weight"]
        assert t.orig_size == 1024 and t.kind == 1 and t.dtype_name == b"bfloat16" and [t.shape[d] for d in range(t.ndim)] == [16, 32]
        idx = (C.c_uint32 * len(ok))(*[i for i, t in enumerate(infos) if t.supported])
        p = C.c_void_p()
        assert L.ptwm_b200_plan_create(h, idx, len(ok), C.byref(p)) == 0
        L.ptwm_b200_plan_destroy(p)
        L.ptwm_b200_close(h)


def test_blake3_and_the_legacy_table_commitment(L):
    """BLAKE3 against the Python package at every tree shape up to a few chunks; the legacy header's hash of the
    Extension Table (container.rs:1299-1301) is checked; a built-in label over a foreign id is not a built-in
    (extension/builtins.rs:283-333)."""
    import blake3
    for n in [0, 1, 63, 64, 65, 1023, 1024, 1025, 2048, 2049, 3073, 4096, 5000, 8193, 100000]:
        data = bytes((i * 7 + 3) & 0xFF for i in range(n))
        out = C.create_string_buffer(32)
        L.ptwm_b200_blake3(data, n, out)
        assert out.raw == blake3.blake3(data).digest(), n
    blob = bytearray(open(os.path.join(GOLD, "reference", "legacy_v1_1_0.ptwm"), "rb").read())
    et_off, et_len = int.from_bytes(blob[11:19], "little"), int.from_bytes(blob[19:27], "little")
    assert bytes(blob[27:59]) == blake3.blake3(bytes(blob[et_off:et_off + et_len])).digest()
    first_label = bytes(blob[et_off + 4 + 34:et_off + 4 + 34 + 16])
    assert first_label == b"io.ptwm.builtin.", first_label
    assert bytes(blob[et_off + 4:et_off + 36]) == blake3.blake3(b"\xBB" * 32 + b"\x00source\x00" + b"1.1.0").digest()
    # a flipped table byte breaks the commitment
    bad = bytearray(blob)
    bad[et_off + 40] ^= 1
    rc, h = _open(L, bytes(bad))
    assert rc < 0 and b"extension table hash mismatch" in L.ptwm_b200_last_error()
    # a foreign id under a built-in label (hash recomputed so that only the id is wrong): every chain uses the
    # first entry (source), so no tensor can be planned any more
    bad = bytearray(blob)
    bad[et_off + 4] ^= 1
    bad[27:59] = blake3.blake3(bytes(bad[et_off:et_off + et_len])).digest()
    rc, h = _open(L, bytes(bad))
    assert rc == 0
    assert not any(t.supported for t in _infos(L, h))
    L.ptwm_b200_close(h)


def test_legacy_reader_survives_mutations_and_truncation(L):
    """Every byte of the header, tables, registry and index flipped, a sample of the record bytes flipped, and every
    7th truncation: the legacy reader answers (error or success) and never reads outside the buffer."""
    blob = bytearray(open(os.path.join(GOLD, "reference", "legacy_v1_0_0_native.ptwm"), "rb").read())
    et_off, et_len = (int.from_bytes(blob[o:o + 8], "little") for o in (11, 19))
    idx_off, pre_off, pre_len = (int.from_bytes(blob[o:o + 8], "little") for o in (59, 75, 83))
    spots = set(range(0, 91)) | set(range(et_off, et_off + et_len, 3)) | set(range(pre_off, pre_off + pre_len)) | set(range(idx_off, len(blob)))
    spots |= set(range(pre_off + pre_len, idx_off, 5))
    rejected = 0
    for i in sorted(spots):
        m = bytearray(blob)
        m[i] ^= 0xA5
        rc, h = _open(L, bytes(m))
        if rc < 0:
            rejected += 1
        else:
            L.ptwm_b200_close(h)
    assert rejected > 50
    for cut in range(0, len(blob), 7):
        rc, h = _open(L, bytes(blob[:cut]))
        assert rc < 0


def test_bad_magic_and_short_input(L):
    for blob in (b"", b"\x89PT", b"not a container at all", b"\x89PTWM\r\n\x1a\n" + b"\x00" * 64):
        rc, h = _open(L, blob if blob else b"\x00")
        assert rc < 0


def test_contiguous_shards_cover_everything():
    rng = np.random.default_rng(1)
    costs = list(rng.integers(1, 1000, 291))
    for world in (1, 2, 4, 8):
        parts = contiguous_shards(costs, world)
        assert [i for p in parts for i in p] == list(range(len(costs)))
        sums = [sum(costs[i] for i in p) for p in parts]
        assert max(sums) <= sum(costs) / world + max(costs)
    infos = [dict(compressed=10, orig_size=20)] * 5
    assert sum((shard_for_rank(infos, r, 2) for r in range(2)), []) == [0, 1, 2, 3, 4]


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()


def test_malformed_per_plane_op_chains_are_rejected(L, monkeypatch):
    """Chains that hang IntDelta / MantissaZeroStrip nodes off a byte split in ways the production builders never do:
    both the oracle and the library's parser refuse them (an error or an unsupported tensor), neither guesses."""
    import numpy as np
    import oracle
    raw = (np.arange(4096, dtype=np.uint16) & 0xFFF0).tobytes()
    spec = oracle.TensorSpec("_", oracle.DT_BF16, [4096], raw, post={1: ("intdelta",)})
    kind, nodes, edges, terms = oracle.chain_graph(spec)
    good = oracle.write_compact(spec, emit_hash=True)
    assert oracle.decode_compact(good)[0] == raw
    rc, h = _open(L, good)
    assert rc == 0 and _infos(L, h)[0].supported
    L.ptwm_b200_close(h)
    split = 2
    cases = {
        "plane out of range": (nodes, edges[:2] + [(split, 5, 3, 0)], terms),
        "op fed from before the split": (nodes, edges[:2] + [(1, 0, 3, 0)], terms),
        "terminal skips the op": (nodes, edges, [terms[0], (split, 1, terms[1][2])]),
        "terminal on the wrong output": (nodes, edges, [terms[0], (3, 1, terms[1][2])]),
        "two ops on one plane": (nodes + [(oracle.OP_INTDELTA, b"")], edges + [(split, 1, 4, 0)], terms),
        "op chained on an op": (nodes + [(oracle.OP_INTDELTA, b"")], edges + [(3, 0, 4, 0)], [terms[0], (4, 0, terms[1][2])]),
        "strip of zero bits": (nodes[:3] + [(oracle.OP_MZS, b"\x00")], edges, terms),
        "strip of eight bits": (nodes[:3] + [(oracle.OP_MZS, b"\x08")], edges, terms),
        "strip without its parameter": (nodes[:3] + [(oracle.OP_MZS, b"")], edges, terms),
        "delta with a parameter": (nodes[:3] + [(oracle.OP_INTDELTA, b"\x01")], edges, terms),
    }
    for what, graph in cases.items():
        monkeypatch.setattr(oracle, "chain_graph", lambda s, g=graph: (kind, list(g[0]), list(g[1]), list(g[2])))
        frame = oracle.write_compact(spec, emit_hash=True)
        with pytest.raises(oracle.OracleError):
            oracle.decode_compact(frame)
        rc, h = _open(L, frame)
        if rc == 0:
            assert not _infos(L, h)[0].supported, what
            L.ptwm_b200_close(h)


def test_sharded_open_partitions_the_records(L):
    """ptwm_b200_open_shard reads the records of one rank's contiguous run only; the runs of all ranks partition
    the container and agree with the cut by record bytes."""
    import oracle
    from _data import mixed_model
    specs = mixed_model()
    blob = oracle.write_container(specs, chunk_size=4096, emit_crc=True)
    buf = (C.c_char * len(blob)).from_buffer_copy(blob)
    rc, h = _open(L, blob)
    assert rc == 0
    full = _infos(L, h)
    names = [t.name for t in full]
    sizes = {t.name: (t.orig_size, t.first_byte, t.end_byte) for t in full}
    L.ptwm_b200_close(h)
    for world in (1, 2, 3, 5, len(specs) + 3):
        seen = []
        for rank in range(world):
            hs = C.c_void_p()
            assert L.ptwm_b200_open_shard(C.addressof(buf), len(blob), rank, world, C.byref(hs)) == 0
            infos = _infos(L, hs)
            assert [t.name for t in infos] == names
            mine = [i for i, t in enumerate(infos) if t.supported]
            assert mine == list(range(mine[0], mine[-1] + 1)) if mine else True
            for i in mine:
                assert (infos[i].orig_size, infos[i].first_byte, infos[i].end_byte) == sizes[infos[i].name]
            for i, t in enumerate(infos):
                if i not in mine:
                    assert b"another rank" in t.unsupported_reason and t.compressed > 0
            if mine:
                idx = (C.c_uint32 * len(mine))(*mine)
                p = C.c_void_p()
                assert L.ptwm_b200_plan_create(hs, idx, len(mine), C.byref(p)) == 0
                L.ptwm_b200_plan_destroy(p)
            seen += mine
            L.ptwm_b200_close(hs)
        assert seen == list(range(len(names))), world
    hs = C.c_void_p()
    assert L.ptwm_b200_open_shard(C.addressof(buf), len(blob), 2, 2, C.byref(hs)) < 0


def test_shared_state_fit_on_the_host(L):
    """Pass 2 of the writer without a GPU.  One plane: the shared state is the state the codec fits to that plane
    (the oracle's, pinned by the reference's fixtures).  Planes that behave alike: one state, fitted to their pooled
    counts.  Two families over the same symbols that behave differently: two states."""
    rng = np.random.default_rng(9)
    slow = lambda rows: (120 + np.cumsum(rng.random((rows, 256)) < 0.06, axis=1) % 4).astype(np.uint8).tobytes()
    noise = lambda rows: (120 + rng.integers(0, 4, (rows, 256))).astype(np.uint8).tobytes()
    a = slow(64)
    st, sv, _ = oracle.plane_encode(oracle.O1SAC, a, 256)
    assert sv == 1 and _lib.fit_shared_states_host([a], [256]) == [st]
    b, c = slow(80), slow(48)
    pooled, _, _ = oracle.plane_encode(oracle.O1SAC, a + b + c, 256)
    assert _lib.fit_shared_states_host([a, b, c], [256, 256, 256]) == [pooled]
    planes = [slow(200), noise(200), slow(220), noise(180), slow(190), noise(210)]
    states = _lib.fit_shared_states_host(planes, [256] * 6)
    assert len(states) == 2
    # each state is the fit of one family's pooled counts, in the order of the families' first planes
    assert states[0] == oracle.plane_encode(oracle.O1SAC, planes[0] + planes[2] + planes[4], 256)[0]
    assert states[1] == oracle.plane_encode(oracle.O1SAC, planes[1] + planes[3] + planes[5], 256)[0]
    assert _lib.fit_shared_states_host([], []) == []
