"""Parity of the CUDA decode path with the CPU oracle, through the C ABI.

Bit-exact is the bar: every comparison is on raw bytes."""
import ctypes as C
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import oracle
import ptwm_b200
from ptwm_b200 import _lib
from _data import mixed_model, spec_bf16, spec_f32, specs_fp8, specs_nvfp4

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")

# canonical ids of the built-in codecs: blake3([0xBB]*32 | 0 | name | 0 | "1.1.0") (extension/id.rs:21-31)
IDS = {
    oracle.IDENTITY: "fc2dea1265e3394c57c2df3b868b732ccaa1ee876bd4b1ce27d38f842c6112b5",
    oracle.HUFFMAN: "614155b5a8c9efb689219bcca3cbf7855e29d3023208ce61cca7a36849248e33",
    oracle.RANS: "39c875ef9793a9c5ebe199116debac4c9d5388b8b7cf2fe6b575845f0ca1624e",
    oracle.TANS: "e4868545e7b22282695972441494e70569ab27595d19349114e852125d96daa4",
    oracle.O1SAC: "0b8426e0a670d114f24ee4614837c9578ff3034f11e4e9e9c0f5d92a49887770",
}


def bytes_of(t: torch.Tensor) -> bytes:
    return t.contiguous().view(torch.uint8).cpu().numpy().tobytes()


def dispatch_decode(codec, payload: bytes, decoded_len: int, state: bytes = b"", sv: int = 0, symbol="ptwm_hardware_backend_v1_dispatch_decode_cuda"):
    """One plane payload through the reference-facing symbol."""
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    src = torch.frombuffer(bytearray(payload), dtype=torch.uint8).to(dev) if payload else torch.empty(0, dtype=torch.uint8, device=dev)
    out = torch.full((max(decoded_len, 1) + 64,), 0xAB, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    st = C.create_string_buffer(state, len(state)) if state else None
    rc = getattr(L, symbol)(sv, st, len(state), bytes.fromhex(IDS[codec]), 32, src.data_ptr() if payload else 0, len(payload), out.data_ptr(), decoded_len, 0)
    return rc, bytes_of(out[:max(rc, 0)]), bytes_of(out[decoded_len:decoded_len + 64])


def plane_cases():
    rng = np.random.default_rng(7)
    sizes = [1, 2, 3, 4, 5, 7, 8, 9, 31, 32, 33, 100, 1023, 4093, 4096, 65536, 100003, 262144]
    for n in sizes:
        yield "gauss", ((rng.normal(0, 3, n).astype(np.int64) + 120) % 256).astype(np.uint8).tobytes()
        yield "two", rng.integers(0, 2, n, dtype=np.uint8).tobytes()
        yield "const", np.full(n, 7, np.uint8).tobytes()
        yield "nibble", rng.integers(0, 16, n, dtype=np.uint8).tobytes()
    yield "wide", (np.arange(256 * 40) % 256).astype(np.uint8).tobytes() + bytes(9000)
    yield "skew", np.concatenate([np.zeros(200000, np.uint8), rng.integers(0, 256, 3000, dtype=np.uint8)]).tobytes()
    yield "random", rng.integers(0, 256, 50000, dtype=np.uint8).tobytes()
    yield "empty", b""


@pytest.mark.parametrize("codec", [oracle.IDENTITY, oracle.HUFFMAN, oracle.RANS, oracle.TANS])
def test_plane_payloads_match_oracle(codec):
    coded = 0
    for tag, plane in plane_cases():
        st, sv, payload = oracle.plane_encode(codec, plane)
        assert oracle.plane_decode(codec, payload, len(plane)) == plane
        rc, got, guard = dispatch_decode(codec, payload, len(plane))
        assert rc == len(plane), (tag, len(plane), rc, _lib.last_error())
        assert got == plane, (tag, len(plane), next(i for i in range(len(plane)) if got[i] != plane[i]))
        assert guard == b"\xAB" * 64, (tag, len(plane), "wrote past the plane")
        coded += codec != oracle.IDENTITY and payload[:1] == b"\x01"
    if codec != oracle.IDENTITY:
        assert coded > 20


def test_o1sac_payloads_match_oracle():
    rng = np.random.default_rng(8)
    for rows, rl in [(1, 1), (3, 7), (32, 32), (64, 256), (500, 128)]:
        walk = (np.cumsum(rng.integers(-1, 2, (rows, rl)), axis=1) + 120).astype(np.uint8).tobytes()
        st, sv, payload = oracle.plane_encode(oracle.O1SAC, walk, 0)  # the flat ABI carries no layout: one row
        rc, got, guard = dispatch_decode(oracle.O1SAC, payload, len(walk), st, sv, symbol="ptwm_plane_codec_v1_decode_cuda")
        assert rc == len(walk), _lib.last_error()
        assert got == walk and guard == b"\xAB" * 64


def test_host_buffer_pair_decodes_rans():
    plane = ((np.random.default_rng(9).normal(0, 2, 30000).astype(np.int64) + 100) % 256).astype(np.uint8).tobytes()
    _, _, payload = oracle.plane_encode(oracle.RANS, plane)
    out = C.create_string_buffer(len(plane))
    rc = _lib.lib().ptwm_plane_codec_v1_decode(payload, len(payload), out, len(plane))
    assert rc == len(plane) and out.raw == plane
    small = C.create_string_buffer(10)
    assert _lib.lib().ptwm_plane_codec_v1_decode(payload, len(payload), small, 10) == -2  # BufferTooSmall (native.rs:634-657)


def test_payload_produced_on_a_side_stream_is_ordered_by_the_stream_handle():
    """The reference hands the library's stream handle to the tensor's DLPack export, which makes that stream wait
    for the producer (flavor/native.rs:105-112, crates/ptwm-py/src/hardware.rs:119-126).  Nothing else orders the two:
    no device-wide synchronisation happens between producing the payload and the call."""
    L = _lib.lib()
    plane = ((np.random.default_rng(12).normal(0, 3, 200000).astype(np.int64) + 120) % 256).astype(np.uint8).tobytes()
    for codec, symbol in ((oracle.RANS, "ptwm_hardware_backend_v1_dispatch_decode_cuda"), (oracle.HUFFMAN, "ptwm_plane_codec_v1_decode_cuda"),
                          (oracle.TANS, "ptwm_b200_decode_plane_noalloc")):
        _, _, payload = oracle.plane_encode(codec, plane)
        assert payload[:1] == b"\x01"
        staged = torch.frombuffer(bytearray(payload), dtype=torch.uint8).pin_memory()
        src = torch.zeros(len(payload), dtype=torch.uint8, device="cuda")  # reads as a raw-tagged payload until the producer has run
        out = torch.zeros(len(plane), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        handle = L.ptwm_hardware_backend_v1_cuda_stream_handle(0)
        side = torch.cuda.Stream()  # a non-blocking stream, like every torch side stream
        with torch.cuda.stream(side):
            torch.cuda._sleep(400_000_000)  # the producer is still busy when the call below starts
            src.copy_(staged, non_blocking=True)
        torch.cuda.ExternalStream(handle).wait_stream(side)  # what __dlpack__(stream=handle) does
        args = [1, None, 0, bytes.fromhex(IDS[codec]), 32, src.data_ptr(), len(payload), out.data_ptr(), len(plane), 0]
        if symbol.endswith("noalloc"):
            args.append(handle)
        rc = getattr(L, symbol)(*args)
        assert rc == len(plane), (symbol, rc, _lib.last_error())
        assert bytes_of(out) == plane, symbol


def test_stream_handle_is_persistent():
    L = _lib.lib()
    a = L.ptwm_hardware_backend_v1_cuda_stream_handle(0)
    assert a != 0 and a == L.ptwm_hardware_backend_v1_cuda_stream_handle(0) == L.ptwm_plane_codec_v1_cuda_stream_handle(0)


def test_unknown_codec_id_is_unsupported():
    L = _lib.lib()
    out = torch.empty(16, dtype=torch.uint8, device="cuda")
    rc = L.ptwm_hardware_backend_v1_dispatch_decode_cuda(0, None, 0, bytes(32), 32, out.data_ptr(), 4, out.data_ptr(), 4, 0)
    assert rc == -5


# ---- containers -------------------------------------------------------------
def check_container(blob: bytes, expected: dict, verify=True):
    h = ptwm_b200.ContainerHandle(blob, device=0, verify=verify)
    got = dict(h.decode_model())
    assert list(got) == list(expected)
    for name, raw in expected.items():
        g = bytes_of(got[name])
        assert len(g) == len(raw), name
        if g != raw:
            first = next(i for i in range(len(raw)) if g[i] != raw[i])
            raise AssertionError(f"{name}: first mismatch at byte {first} of {len(raw)}")
    # the streamed form (host copy, pieces decoded while later bytes are still being copied) gives the same tensors
    for pieces in (1, 3):
        streamed = dict(h.decode_model_streamed(pieces=pieces))
        assert list(streamed) == list(expected)
        for name, raw in expected.items():
            assert bytes_of(streamed[name]) == raw, (name, pieces)
    return h, got


CONTAINER_CASES = {
    "whole": dict(),
    "chunk4k_crc": dict(chunk_size=4096, emit_crc=True),
    "chunk1000_hash_crc": dict(chunk_size=1000, emit_hash=True, emit_crc=True),
    "chunk64k": dict(chunk_size=65536, emit_crc=True),
    "huffman_8k": dict(forced_codec=oracle.HUFFMAN, chunk_size=8192, emit_crc=True, emit_hash=True),
    "rans_8k": dict(forced_codec=oracle.RANS, chunk_size=8192, emit_crc=True, emit_hash=True),
    "tans_8k": dict(forced_codec=oracle.TANS, chunk_size=8192, emit_crc=True),
    "identity": dict(forced_codec=oracle.IDENTITY, emit_crc=True, emit_hash=True),
    "menu_hr_o1": dict(menu=(oracle.HUFFMAN, oracle.RANS, oracle.O1SAC), emit_crc=True, emit_hash=True),
    "menu_hr_chunk_odd": dict(menu=(oracle.HUFFMAN, oracle.RANS), chunk_size=777),
}


@pytest.mark.parametrize("case", list(CONTAINER_CASES))
def test_mixed_model_matches_oracle(case):
    specs = mixed_model()
    blob = oracle.write_container(specs, **CONTAINER_CASES[case])
    oc = oracle.Container(blob)
    expected = {s.name: oc.decode(i) for i, s in enumerate(specs)}
    assert all(expected[s.name] == s.raw for s in specs)
    h, got = check_container(blob, expected)
    # typed views: dtype and shape follow the record (python/ptwm/core/_decompressor.py:141-160)
    assert got["blk.q.weight"].dtype == torch.bfloat16 and list(got["blk.q.weight"].shape) == list(specs[0].shape)
    assert got["blk.gate.f32"].dtype == torch.float32 and got["blk.fp8.weight"].dtype == torch.float8_e4m3fn
    # random access agrees with the batched pass (ContainerReader::decode_tensor)
    for name in ("blk.k.weight", "blk.nv.weight_scale", "odd.bf16", "scalar.f32", "empty.f32"):
        assert bytes_of(h.decode(name)) == expected[name]


def test_committed_goldens():
    man = json.load(open(os.path.join(GOLD, "oracle", "manifest.json")))
    for name, meta in man.items():
        if name == "frames":
            for fn, (n, sha) in meta.items():
                t = ptwm_b200.Decompressor(ptwm_b200.DecompressionConfig(device=0)).decompress(open(os.path.join(GOLD, "oracle", fn), "rb").read())
                raw = bytes_of(t)
                assert len(raw) == n and hashlib.sha256(raw).hexdigest() == sha, fn
            continue
        h = ptwm_b200.ContainerHandle(open(os.path.join(GOLD, "oracle", name + ".ptwm"), "rb").read(), device=0)
        for tname, t in h.decode_model():
            raw = bytes_of(t)
            n, sha = meta["tensors"][tname]
            assert len(raw) == n and hashlib.sha256(raw).hexdigest() == sha, (name, tname)


def test_reference_fixtures_on_gpu():
    # the reference's own files: Identity planes with hash + CRC, and every supported \x89PTWS seed
    import xxhash
    ref = os.path.join(GOLD, "reference")
    blob = open(os.path.join(ref, "ptwc_bound_source"), "rb").read()
    h = ptwm_b200.ContainerHandle(blob, device=0)
    oc = oracle.Container(blob)
    for i, (name, t) in enumerate(h.decode_model()):
        assert bytes_of(t) == oc.decode(i)
    assert xxhash.xxh64(bytes_of(h.decode("t1"))).hexdigest() == json.load(open(os.path.join(ref, "expected.json")))["ptwc_bound_source"]["t1"][1]
    done, delta = 0, 0
    for f in sorted(os.listdir(os.path.join(ref, "compact_decode"))):
        frame = b"\x89PTWS" + open(os.path.join(ref, "compact_decode", f), "rb").read()
        try:
            want, _ = oracle.decode_compact(frame)
        except oracle.OracleError:
            continue  # zstd planes: outside the hot path
        got = ptwm_b200.Decompressor(ptwm_b200.DecompressionConfig(device=0)).decompress(frame)
        assert bytes_of(got) == want, f
        done += 1
        delta += "smooth" in f or "byte_bf16" in f
    assert done >= 16 and delta == 7  # the seven split + IntDelta seeds carry the reference's own hashes and plane CRCs


def test_integrity_checks_fire():
    specs = [spec_bf16("w", 64, 256, 1)]
    for kw, needle in ((dict(emit_crc=True, chunk_size=4096), "CRC"), (dict(emit_hash=True), "hash")):
        blob = bytearray(oracle.write_container(specs, forced_codec=oracle.IDENTITY, **kw))
        h = ptwm_b200.ContainerHandle(bytes(blob), device=0)
        inf = h.tensor_infos()[0]
        blob[inf["end_byte"] - 3] ^= 0x10  # flip a stored mantissa-or-exponent byte: decodes, but to other values
        bad = ptwm_b200.ContainerHandle(bytes(blob), device=0)
        with pytest.raises(ptwm_b200.PtwmError, match=needle):
            bad.decode_model()
        assert len(ptwm_b200.ContainerHandle(bytes(blob), device=0, verify=False).decode_model()) == 1


def test_full_size_properties():
    # BASELINE-sized tensors: too slow for the serial oracle decode of every case, so check through
    # self-verifying containers (hash + CRC) and against the source bytes.
    specs = [spec_bf16("c1.bf16", 4096, 4096, 0), spec_f32("c2.f32", 4096, 1024, 1)] + specs_fp8("c3", 2048, 4096, 2) + specs_nvfp4("c4", 1024, 4096, 3)
    for kw in (dict(chunk_size=65536, emit_crc=True, emit_hash=True, menu=(oracle.IDENTITY, oracle.HUFFMAN, oracle.RANS, oracle.O1SAC)),
               dict(chunk_size=32768, forced_codec=oracle.HUFFMAN, emit_crc=True)):
        blob = oracle.write_container(specs, **kw)
        check_container(blob, {s.name: s.raw for s in specs})


def test_replica_mode_with_one_rank_equals_decode_model():
    # the gather-of-one path: the rank's own span is the whole range, nothing crosses NVLink, then one local decode
    from ptwm_b200.sharding import decode_replica
    specs = mixed_model()
    blob = oracle.write_container(specs, chunk_size=4096, emit_crc=True, emit_hash=True)
    h = ptwm_b200.ContainerHandle(torch.frombuffer(bytearray(blob), dtype=torch.uint8).pin_memory(), device=0)
    got, received = decode_replica(h)
    assert received == 0 and [n for n, _ in got] == [s.name for s in specs]
    for (name, t), s in zip(got, specs):
        assert bytes_of(t) == s.raw, name
    some, _ = decode_replica(h, names=[specs[3].name, specs[0].name])
    assert [n for n, _ in some] == [specs[3].name, specs[0].name] and bytes_of(some[0][1]) == specs[3].raw


def test_partial_blob_span_and_subset_plan():
    # a rank keeps only the byte range of its own tensors on the device
    specs = mixed_model()
    blob = oracle.write_container(specs, chunk_size=4096, emit_crc=True)
    h = ptwm_b200.ContainerHandle(blob, device=0)
    infos = h.tensor_infos()
    from ptwm_b200.sharding import shard_for_rank
    seen = []
    for rank in range(3):
        idx = shard_for_rank(infos, rank, 3)
        seen += idx
        plan = h.plan(idx)
        lo, hi = plan.blob_span
        part = torch.frombuffer(bytearray(blob[lo:hi]), dtype=torch.uint8).cuda() if hi > lo else torch.empty(0, dtype=torch.uint8, device="cuda")
        out = torch.empty(plan.out_bytes, dtype=torch.uint8, device="cuda")
        scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device="cuda")
        plan.run(part, out, scratch, blob_first=lo, flags=ptwm_b200.VERIFY_CRC)
        for i, v in zip(idx, plan.views(out)):
            assert bytes_of(v) == specs[i].raw, specs[i].name
    assert seen == list(range(len(specs)))


# ---- planes that leave the fast paths -------------------------------------------------------
def _hard_plane(n, seed):
    """Exponent-plane bytes with long runs of rare symbols: rANS groups that need more than
    eight renormalisation bytes, Huffman codes longer than the table window, and enough distinct
    symbols in some chunks to leave the per-lane symbol lists."""
    rng = np.random.default_rng(seed)
    plane = ((rng.normal(0, 1.2, n).astype(np.int64) + 120) % 256).astype(np.uint8)
    for start in range(1000, n - 600, 9000):          # bursts of (nearly) uniform bytes inside a peaked chunk
        plane[start:start + 500] = rng.integers(0, 256, 500, dtype=np.uint8)
    plane[n // 2:n // 2 + 70000] = rng.integers(0, 48, 70000, dtype=np.uint8) * 5   # a chunk with 48 distinct symbols
    return plane.tobytes()


@pytest.mark.parametrize("codec", [oracle.RANS, oracle.HUFFMAN, oracle.TANS])
@pytest.mark.parametrize("offset", [0, 3])
def test_fused_16bit_leaves_and_reenters_the_fast_loops(codec, offset):
    n = 5 * 65536 + 12345
    low = np.random.default_rng(11).integers(0, 256, n, dtype=np.uint8).tobytes()
    raw = oracle.merge_inverse(oracle.M16, [low, _hard_plane(n, 5)])
    specs = []
    if offset:  # an odd-sized neighbour shifts every later payload in the file to another alignment
        specs.append(oracle.TensorSpec("pad", oracle.DT_U8, [offset], bytes(range(offset))))
    specs.append(oracle.TensorSpec("w", oracle.DT_BF16, [n], raw))
    blob = oracle.write_container(specs, chunk_size=65536, forced_codec=codec)
    check_container(blob, {s.name: s.raw for s in specs})


@pytest.mark.parametrize("case", [dict(forced_codec=oracle.RANS, chunk_size=65536), dict(forced_codec=oracle.HUFFMAN, chunk_size=20001, emit_crc=True),
                                  dict(menu=(oracle.HUFFMAN, oracle.RANS), chunk_size=32768, emit_hash=True), dict(forced_codec=oracle.RANS, chunk_size=20001),
                                  dict(forced_codec=oracle.TANS, chunk_size=20001, emit_crc=True), dict(forced_codec=oracle.TANS, chunk_size=65536),
                                  dict(forced_codec=oracle.TANS, chunk_size=4099)])
def test_larger_mixed_model_runs_the_round_loops(case):
    """Tensors of several chunks each, chunk sizes that leave every stream and partner plane at an odd address:
    the 32- and 16-element round loops of the 16-bit, fp8 and fp32 paths, their heads and tails."""
    specs = mixed_model(scale=4)
    blob = oracle.write_container(specs, **case)
    check_container(blob, {s.name: s.raw for s in specs})


@pytest.mark.parametrize("fixture", ["legacy_v1_1_0", "legacy_v1_0_0", "legacy_v1_0_0_native"])
def test_legacy_fixtures_decode_to_the_reference_hashes(fixture):
    """crates/ptwm-core/tests/legacy_fixtures.rs:65-123: the tensors of the legacy fixtures that lie on the hot path
    (Order1ScaleAC scale planes with a shared prelude state, a two-chunk tANS plane) against the reference's table."""
    blob = open(os.path.join(GOLD, "reference", fixture + ".ptwm"), "rb").read()
    exp = json.load(open(os.path.join(GOLD, "reference", "expected.json")))[fixture]
    h = ptwm_b200.ContainerHandle(blob, device=0)
    assert h.layout == "legacy"
    names = [t["name"] for t in h.tensor_infos() if t["supported"]]
    assert "model.layers.2.chunked.weight" in names and ("native" in fixture or "model.layers.0.q.scale" in names)
    for name, t in h.decode_model(names):
        raw = bytes_of(t)
        n, want = exp[name]
        assert len(raw) == n and oracle.xxh64(raw) == int(want, 16), name
    assert list(h.decode("model.layers.2.chunked.weight").shape) == [16, 32]


def _post_specs(n: int):
    rng = np.random.default_rng(n)
    smooth = (np.cumsum(rng.standard_normal(n)) * 0.01).astype(np.float32)
    bf = (smooth.view(np.uint32) >> 16).astype(np.uint16)
    quant = (bf & 0xFFF8).astype(np.uint16)  # three low mantissa bits zero, as after dequantising a 4-bit mantissa
    return [oracle.TensorSpec("delta.bf16", oracle.DT_BF16, [n], bf.tobytes(), post={1: ("intdelta",)}),
            oracle.TensorSpec("strip.bf16", oracle.DT_BF16, [n // 4, 4], quant.tobytes(), post={0: ("mzs", 3)}),
            oracle.TensorSpec("delta.f32", oracle.DT_F32, [n], smooth.tobytes(), post={3: ("intdelta",)}),
            oracle.TensorSpec("both.f32", oracle.DT_F32, [n], (smooth.view(np.uint32) & 0xFFFFFF00).astype(np.uint32).tobytes(), post={0: ("mzs", 7), 3: ("intdelta",)}),
            oracle.TensorSpec("two.bf16", oracle.DT_BF16, [n], quant.tobytes(), post={0: ("mzs", 2), 1: ("intdelta",)}),
            oracle.TensorSpec("plain.bf16", oracle.DT_BF16, [n], bf.tobytes())]


@pytest.mark.parametrize("n,opts", [(5000, dict()), (5000, dict(chunk_size=1000, emit_crc=True, emit_hash=True)),
                                    (100_004, dict(forced_codec=oracle.RANS, chunk_size=8192, emit_crc=True)),
                                    (100_004, dict(forced_codec=oracle.HUFFMAN, chunk_size=32768, emit_crc=True, emit_hash=True)),
                                    (70_000, dict(forced_codec=oracle.TANS, chunk_size=65536, emit_crc=True)),
                                    (4_300_000, dict(forced_codec=oracle.IDENTITY, emit_crc=True, emit_hash=True))])
def test_per_plane_ops_match_oracle(n, opts):
    # IntDelta on the exponent plane, MantissaZeroStrip on a mantissa plane (python/ptwm/preprocessing/_chains.py:360-389,486-560);
    # the largest case spans more than 256 tiles of the running sum
    specs = _post_specs(n)
    blob = oracle.write_container(specs, **opts)
    h, got = check_container(blob, {s.name: s.raw for s in specs})
    # a wrong CRC of a terminal plane is noticed
    if opts.get("emit_crc") and n <= 5000:
        oc = oracle.Container(blob)
        p = oc.tensors[0]["planes"][1]
        bad = bytearray(blob)
        bad[p["payload_off"] + p["payload_len"] - 1] ^= 0x10
        with pytest.raises(ptwm_b200.PtwmError):
            ptwm_b200.ContainerHandle(bytes(bad), device=0).decode_model()
    for s in specs[:3]:
        frame = oracle.write_compact(s, emit_hash=True)
        assert bytes_of(ptwm_b200.Decompressor(ptwm_b200.DecompressionConfig(device=0)).decompress(frame)) == s.raw


def test_prefetched_handle_decodes_the_same():
    # the copy of a pinned container to the GPU starts before the parse; streamed and random-access decodes use it
    specs = mixed_model()
    blob = oracle.write_container(specs, chunk_size=4096, emit_crc=True, emit_hash=True)
    pinned = torch.empty(len(blob), dtype=torch.uint8, pin_memory=True)
    pinned.copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8))
    for pieces in (1, 4):
        h = ptwm_b200.ContainerHandle(pinned, device=0, prefetch=True)
        assert h._prefetch is not None
        got = dict(h.decode_model_streamed(pieces=pieces))
        assert all(bytes_of(got[s.name]) == s.raw for s in specs)
        some = [specs[2].name, specs[5].name]
        part = dict(h.decode_model_streamed(names=some, pieces=2))
        assert all(bytes_of(part[n]) == next(s.raw for s in specs if s.name == n) for n in some)
    h = ptwm_b200.ContainerHandle(pinned, device=0, prefetch=True)
    assert bytes_of(h.decode(specs[0].name)) == specs[0].raw
    # pageable memory: the option is ignored
    assert ptwm_b200.ContainerHandle(blob, device=0, prefetch=True)._prefetch is None


def test_tans_full_size_planes():
    # four bf16 [4096,4096] tensors (BASELINE config C1's shape) with tANS forced on every plane, 64 KiB chunks:
    # 1024 tANS streams of 65536 symbols, the case the tANS profile summary was captured on
    specs = []
    for i in range(4):
        w = (torch.randn(4096, 4096, generator=torch.Generator().manual_seed(i)) * 0.02).to(torch.bfloat16)
        specs.append(oracle.TensorSpec(f"w{i}", oracle.DT_BF16, [4096, 4096], w.view(torch.uint8).numpy().tobytes()))
    blob = oracle.write_container(specs, chunk_size=65536, forced_codec=oracle.TANS)
    h = ptwm_b200.ContainerHandle(blob, device=0, verify=False)
    assert any(c == oracle.TANS for t in oracle.Container(blob).tensors for c in [p["codec"] for p in t["planes"]])
    for (name, t), s in zip(h.decode_model(), specs):
        assert name == s.name and bytes_of(t) == s.raw


@pytest.mark.parametrize("seed", range(12))
def test_random_containers(seed):
    """Seeded random state dicts: tensor count, dtypes, shapes (odd sizes, so streams and partner planes land on
    every alignment), chunk size, codec and integrity fields all drawn at random; decoded bytes equal the source."""
    rng = np.random.default_rng(1000 + seed)
    specs = []
    for t in range(int(rng.integers(2, 6))):
        kind = ["bf16", "f16", "f32", "fp8", "u8", "bf16"][int(rng.integers(0, 6))]
        rows, cols = int(rng.integers(1, 160)), int(rng.integers(1, 3000))
        if kind == "bf16":
            specs.append(spec_bf16(f"t{t}.bf16", rows, cols, seed * 10 + t, sigma_rows=bool(rng.integers(0, 2))))
        elif kind == "f16":
            w = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(seed * 10 + t)) * 0.02).to(torch.float16)
            specs.append(oracle.TensorSpec(f"t{t}.f16", oracle.DT_F16, [rows, cols], w.view(torch.uint8).numpy().tobytes()))
        elif kind == "f32":
            specs.append(spec_f32(f"t{t}.f32", rows, cols, seed * 10 + t))
        elif kind == "fp8":
            specs += specs_fp8(f"t{t}.fp8", rows, cols, seed * 10 + t)
        else:
            n = rows * cols
            specs.append(oracle.TensorSpec(f"t{t}.u8", oracle.DT_U8, [n], ((rng.normal(0, 2.5, n).astype(np.int64) + 100) % 256).astype(np.uint8).tobytes()))
    case = dict(chunk_size=int(rng.choice([777, 4099, 8192, 20001, 32768, 65536])), emit_crc=bool(rng.integers(0, 2)), emit_hash=bool(rng.integers(0, 2)))
    pick = int(rng.integers(0, 5))
    if pick < 3:
        case["forced_codec"] = [oracle.RANS, oracle.HUFFMAN, oracle.TANS][pick]
    elif pick == 3:
        case["menu"] = (oracle.HUFFMAN, oracle.RANS, oracle.TANS)
    blob = oracle.write_container(specs, **case)
    check_container(blob, {s.name: s.raw for s in specs})


def test_many_scale_chunks_take_the_low_instruction_coder():
    # more Order1ScaleAC chunks than the launch-size threshold of the decoder: the variant with its tables in shared memory
    rng = np.random.default_rng(77)
    rows, cols = 2304, 512
    walk = (120 + np.cumsum(rng.integers(-1, 2, (rows, cols)), axis=1) // 8 + rng.integers(0, 3, (rows, 1))).clip(0, 254).astype(np.uint8)
    specs = [oracle.TensorSpec("big.scales", oracle.DT_U8, [rows, cols], walk.tobytes(), usage="scale"),
             oracle.TensorSpec("tail.scales", oracle.DT_U8, [3, 100], walk[:3, :100].tobytes(), usage="scale")]
    blob = oracle.write_container(specs, chunk_size=512, forced_codec=oracle.O1SAC)
    h, _ = check_container(blob, {s.name: s.raw for s in specs})
    plan = h.plan()
    out = torch.empty(plan.out_bytes, dtype=torch.uint8, device="cuda:0")
    scratch = torch.empty(max(plan.scratch_bytes, 1), dtype=torch.uint8, device="cuda:0")
    plan.run(h.blob_on_device(), out, scratch, flags=ptwm_b200.TIME_KERNELS)
    assert sum(v[2] for k, v in plan.timings(0).items() if k.startswith("o1sac")) >= 2048


def test_container_already_in_device_memory():
    # what the device encoder leaves behind: parsed from a host copy, decoded from where it lies
    specs = mixed_model()
    blob = oracle.write_container(specs, chunk_size=4096)
    on_device = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    h = ptwm_b200.ContainerHandle(on_device, device=0)
    assert h.blob_on_device().data_ptr() == on_device.data_ptr()
    for (name, t), s in zip(h.decode_model(), specs):
        assert name == s.name and bytes_of(t) == s.raw


def test_sharded_handles_decode_their_share():
    # every rank opens the container with shard=(rank, world): together they decode every tensor once
    specs = mixed_model()
    blob = oracle.write_container(specs, chunk_size=4096, emit_crc=True, emit_hash=True)
    want = {s.name: s.raw for s in specs}
    for world in (2, 3):
        got = {}
        for rank in range(world):
            h = ptwm_b200.ContainerHandle(blob, device=0, shard=(rank, world))
            mine = h.shard_indices()
            for name, t in h.decode_model_streamed(indices=mine, pieces=2):
                assert name not in got
                got[name] = bytes_of(t)
        assert got == want
