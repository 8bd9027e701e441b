"""The CPU oracle against the reference's own known answers and against
independent implementations of the third-party hashes."""
import glob
import json
import os
import zlib

import numpy as np
import pytest
import xxhash

import oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")
REF = os.path.join(GOLD, "reference")


def test_hashes_match_independent_implementations():
    rng = np.random.default_rng(0)
    for n in [0, 1, 3, 4, 7, 8, 31, 32, 33, 63, 64, 65, 100, 4096, 100001]:
        b = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        assert oracle.xxh64(b) == xxhash.xxh64(b, seed=0).intdigest()
        assert oracle.crc32(b) == zlib.crc32(b)


def test_ptwc_bound_source_kat():
    # crates/ptwm-core/tests/ptwc.rs:897-902: four fp32 tensors, Identity planes, hash + CRC
    blob = open(os.path.join(REF, "ptwc_bound_source"), "rb").read()
    c = oracle.Container(blob)
    assert c.names == ["t1", "t2", "t3", "t4"]
    exp = json.load(open(os.path.join(REF, "expected.json")))["ptwc_bound_source"]
    for i, t in enumerate(c.tensors):
        raw = c.decode(i)  # verifies plane CRCs and the payload hash
        assert len(raw) == t["orig_size"] == 8 * (i + 1)
        assert t["has_hash"] and xxhash.xxh64(raw).intdigest() == t["hash"]
    assert xxhash.xxh64(c.decode(0)).hexdigest() == exp["t1"][1]


def test_ptwc_trimmed_matches_legacy_fixture_table():
    # crates/ptwm-core/tests/legacy_fixtures.rs:106-116; planes: identity, zstd, tans, huffman
    if not oracle.install_zstd():
        pytest.skip("system libzstd not available for the zstd planes of the fixture")
    blob = open(os.path.join(REF, "ptwc_trimmed"), "rb").read()
    c = oracle.Container(blob)
    exp = json.load(open(os.path.join(REF, "expected.json")))["ptwc_trimmed"]
    seen = set()
    for i, t in enumerate(c.tensors):
        if t["unsupported"]:
            assert t["name"] == "model.layers.1.q.weight"  # delta-coded: out of the hot path
            continue
        raw = c.decode(i)
        n, h = exp[t["name"]]
        assert len(raw) == n and xxhash.xxh64(raw).hexdigest() == h
        seen.update(p["codec"] for p in t["planes"])
    assert {oracle.IDENTITY, oracle.HUFFMAN, oracle.TANS} <= seen


def test_compact_frames_self_check():
    # fuzz/corpus/compact_decode: *_hash carry xxh64, *_crc carry plane CRC-32s.  The *_smooth and byte_bf16 seeds
    # use the split + IntDelta chains (python/ptwm/preprocessing/_chains.py:360-389): their hashes pin the inverse
    # delta, their CRCs that the checksum covers the terminal's bytes (before the inverse).
    have_zstd = oracle.install_zstd()
    ok, delta = 0, 0
    for f in sorted(glob.glob(os.path.join(REF, "compact_decode", "*"))):
        blob = b"\x89PTWS" + open(f, "rb").read()
        try:
            raw, d = oracle.decode_compact(blob)
        except oracle.OracleError as e:
            assert not have_zstd and "zstd" in str(e), (f, e)
            continue
        ok += 1
        delta += "smooth" in f or "byte_bf16" in f
        with pytest.raises(oracle.OracleError):
            oracle.decode_compact(blob + b"\x00")  # fuzz_targets/compact_decode.rs:50-55
    assert delta == 7 and ok >= 16
    if have_zstd:
        assert ok == 28


def test_per_plane_ops_round_trip_through_the_writer():
    # IntDelta on the exponent plane and MantissaZeroStrip on a mantissa plane, both layouts of the writer
    import numpy as np
    rng = np.random.default_rng(3)
    smooth = (np.cumsum(rng.standard_normal(5000)) * 0.01).astype(np.float32)
    bf = (smooth.view(np.uint32) >> 16).astype(np.uint16)
    quant = (bf & 0xFFF8).astype(np.uint16)  # three low mantissa bits zero, as after dequantising a 4-bit mantissa
    specs = [oracle.TensorSpec("a", oracle.DT_BF16, [5000], bf.tobytes(), post={1: ("intdelta",)}),
             oracle.TensorSpec("b", oracle.DT_BF16, [50, 100], quant.tobytes(), post={0: ("mzs", 3)}),
             oracle.TensorSpec("c", oracle.DT_F32, [5000], smooth.tobytes(), post={3: ("intdelta",)}),
             oracle.TensorSpec("d", oracle.DT_F32, [5000], (smooth.view(np.uint32) & 0xFFFFFF00).tobytes(), post={0: ("mzs", 7), 3: ("intdelta",)}),
             oracle.TensorSpec("e", oracle.DT_BF16, [5000], bf.tobytes())]
    for opts in (dict(), dict(chunk_size=1000, emit_crc=True, emit_hash=True), dict(forced_codec=oracle.RANS, chunk_size=4096, emit_crc=True)):
        c = oracle.Container(oracle.write_container(specs, **opts))
        for i, s in enumerate(specs):
            assert c.decode(i) == s.raw, (s.name, opts)
    for s in specs:
        raw, _ = oracle.decode_compact(oracle.write_compact(s, emit_hash=True))
        assert raw == s.raw
    with pytest.raises(ValueError):
        oracle.write_container([oracle.TensorSpec("x", oracle.DT_BF16, [5000], bf.tobytes(), post={0: ("mzs", 3)})])


def test_huffman_weight_header_bytes():
    # entropy/huffman/weights.rs:102-136: 1-byte header for <=127 symbols, 0x80,n above, 0 = 256
    data = bytes([0] * 50 + [1] * 30 + [2] * 20)
    blob = oracle.raw_compress(oracle.HUFFMAN, data * 4)
    assert blob[0] == 0x80 | 3
    wide = bytes(range(200)) * 40 + bytes([0]) * 8000
    blob = oracle.raw_compress(oracle.HUFFMAN, wide)
    assert blob[0] == 0x80 and blob[1] == 200
    full = bytes(range(256)) * 20 + bytes([7]) * 9000
    blob = oracle.raw_compress(oracle.HUFFMAN, full)
    assert blob[0] == 0x80 and blob[1] == 0


def test_huffman_truncated_jump_table_rejected():
    # entropy/huffman/mod.rs:195-206
    with pytest.raises(oracle.OracleError):
        oracle.raw_decompress(oracle.HUFFMAN, bytes([0x82, 0x11, 1, 2, 3]), 10)


@pytest.mark.parametrize("codec", [oracle.HUFFMAN, oracle.RANS, oracle.TANS])
def test_entropy_roundtrips_reference_unit_inputs(codec):
    # entropy/huffman/mod.rs:48-299, entropy/rans/mod.rs:44-258, entropy/tans/mod.rs:453-581
    rng = np.random.default_rng(1)
    cases = [b"", bytes([5]), bytes([1, 2, 3]), bytes([9] * 4), bytes([1, 1, 2, 2, 3]), bytes(rng.integers(0, 3, 4093, dtype=np.uint8)),
             bytes([42] * 5000), bytes(rng.integers(0, 256, 3000, dtype=np.uint8)), bytes((rng.normal(0, 2, 2 << 20).astype(np.int64) % 256).astype(np.uint8)),
             bytes(range(256)) * 8]
    for data in cases:
        st, sv, payload = oracle.plane_encode(codec, data)
        assert st == b"" and sv == 0
        assert oracle.plane_decode(codec, payload, len(data)) == data
        if data == b"":
            assert payload == b"\x00"
    # single symbol: Huffman and rANS encode it, tANS stores raw (codecs/tans.rs:234-238)
    _, _, p = oracle.plane_encode(codec, bytes([42] * 5000))
    assert p[0] == (0 if codec == oracle.TANS else 1)


def test_rans_normalisation_adjusts_most_frequent_symbol():
    # entropy/rans/compress.rs:72-122: table sums to 2048, every present symbol >= 1
    data = bytes([0] * 30000 + [1] * 10000 + list(range(2, 60)))
    blob = oracle.raw_compress(oracle.RANS, data)
    ms = blob[0]
    freqs = [blob[1 + 2 * i] | blob[2 + 2 * i] << 8 for i in range(ms + 1)]
    assert sum(freqs) == 2048 and all(f >= 1 for f in freqs[:60]) and ms == 59
    assert freqs[0] == max(freqs)


def test_range_coder_pmf_roundtrip_and_o1sac():
    # range_coder.rs:204-261 (skewed PMF) through the Order1ScaleAC wrapper; order1_scale_ac.rs:708-958
    rng = np.random.default_rng(3)
    for rows, rl in [(1, 1), (3, 7), (32, 32), (200, 256)]:
        walk = (np.cumsum(rng.integers(-1, 2, (rows, rl)), axis=1) + 120).astype(np.uint8).tobytes()
        for layout in (rl, 0):
            st, sv, payload = oracle.plane_encode(oracle.O1SAC, walk, layout)
            assert sv == 1 and payload[0] == 0  # leading alignment byte (range_coder.rs:28-41)
            pop = sum(bin(b).count("1") for b in st[:32])
            assert len(st) == 32 + 512 + 512 * pop
            assert oracle.plane_decode(oracle.O1SAC, payload, len(walk), st, sv, row_len=layout) == walk
    with pytest.raises(oracle.OracleError):
        oracle.plane_decode(oracle.O1SAC, payload, 10 ** 9, st, sv)  # order1_scale_ac.rs:449-471


def test_quantize_pmf_sums_and_floors():
    # quantize.rs:13-45
    for counts in ([10] * 16, [0] * 255 + [1000], list(range(256))):
        q = oracle.quantize_pmf(counts, 4096)
        assert sum(q) == 4096 and min(q) >= 1


@pytest.mark.parametrize("kind,mult", [(oracle.M16, 2), (oracle.M32, 4), (oracle.FP8_E4M3, 1), (oracle.FP8_E5M2, 1)])
def test_fused_split_merge_roundtrip(kind, mult):
    # transforms/fusion.rs:525+ incl. the odd trailing 16-bit element (fusion.rs:73-89,165-176)
    rng = np.random.default_rng(4)
    for n in [0, 1, 2, 3, 5, 1000, 4093]:
        raw = rng.integers(0, 256, n * mult, dtype=np.uint8).tobytes()
        planes = oracle.split_forward(kind, raw)
        assert oracle.merge_inverse(kind, planes) == raw
    if kind == oracle.M16:
        v = np.array([0xBF80], np.uint16).tobytes()  # -1.0 bf16: S=1 E=0x7F M=0
        p = oracle.split_forward(kind, v)
        assert p[0] == bytes([0x80]) and p[1] == bytes([0x7F])


def test_committed_oracle_goldens_decode():
    man = json.load(open(os.path.join(GOLD, "oracle", "manifest.json")))
    import hashlib
    for name, meta in man.items():
        if name == "frames":
            for fn, (n, sha) in meta.items():
                raw, _ = oracle.decode_compact(open(os.path.join(GOLD, "oracle", fn), "rb").read())
                assert len(raw) == n and hashlib.sha256(raw).hexdigest() == sha
            continue
        c = oracle.Container(open(os.path.join(GOLD, "oracle", name + ".ptwm"), "rb").read())
        for i, t in enumerate(c.tensors):
            raw = c.decode(i)
            n, sha = meta["tensors"][t["name"]]
            assert len(raw) == n and hashlib.sha256(raw).hexdigest() == sha


def test_writer_reproduces_reference_container_bytes():
    # Re-encoding the tensors of ptwc_bound_source with Identity planes, hash and CRC must give
    # the reference writer's bytes back (layout rules of ptwc.rs / tensor_record_compact.rs / CW2).
    blob = open(os.path.join(REF, "ptwc_bound_source"), "rb").read()
    c = oracle.Container(blob)
    specs = [oracle.TensorSpec(t["name"], t["dtype_code"], t["shape"], c.decode(i)) for i, t in enumerate(c.tensors)]
    again = oracle.write_container(specs, forced_codec=oracle.IDENTITY, emit_hash=True, emit_crc=True)
    assert again == blob


LEGACY_FIXTURES = ("legacy_v1_1_0", "legacy_v1_0_0")


@pytest.mark.parametrize("fixture", LEGACY_FIXTURES)
def test_order1_scale_ac_and_chunked_tans_against_legacy_fixtures(fixture):
    """The reference's legacy fixtures (crates/ptwm-core/tests/legacy_fixtures.rs:65-123): the two scale tensors are
    Order1ScaleAC planes with a shared prelude state and rows of 32, the chunked tensor a bf16 split with a two-chunk
    tANS exponent plane.  Decoding them here must give the hashes the reference's own test expects."""
    import _legacy
    blob = open(os.path.join(REF, fixture + ".ptwm"), "rb").read()
    exp = json.load(open(os.path.join(REF, "expected.json")))[fixture]
    shared, tens = _legacy.shared_states(blob), _legacy.tensors(blob)
    for name in ("model.layers.0.q.scale", "model.layers.0.k.scale"):
        p = tens[name]["planes"][0]
        assert p["codec"] == oracle.O1SAC and p["state_source"] == 2 and p["row_len"] == 32
        st = shared[p["state_info"]]
        assert st["codec"] == oracle.O1SAC
        raw = oracle.plane_decode(oracle.O1SAC, p["payload"], tens[name]["orig_size"], state=st["state"], state_version=st["version"], row_len=32)
        n, h = exp[name]
        assert len(raw) == n and xxhash.xxh64(raw).hexdigest() == h
    t = tens["model.layers.2.chunked.weight"]
    planes = []
    for p in t["planes"]:
        assert p["chunks"] is not None and len(p["chunks"]) == 2
        out = b""
        for k, (off, decoded) in enumerate(p["chunks"]):
            end = p["chunks"][k + 1][0] if k + 1 < len(p["chunks"]) else len(p["payload"])
            frame = p["payload"][off:end]
            state_len = int.from_bytes(frame[1:5], "little")
            out += oracle.plane_decode(p["codec"], frame[5 + state_len:], decoded, state=frame[5:5 + state_len], state_version=frame[0])
        planes.append(out)
    assert {p["codec"] for p in t["planes"]} == {oracle.IDENTITY, oracle.TANS}
    raw = oracle.merge_inverse(oracle.M16, planes)
    n, h = exp["model.layers.2.chunked.weight"]
    assert len(raw) == n and xxhash.xxh64(raw).hexdigest() == h
