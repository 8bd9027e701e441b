"""The device encoder against the CPU oracle: forced-codec containers must be
byte-identical to what the oracle's writer (a restatement of the reference's
compressor) produces, selected-codec containers must decode in the oracle
and stay within 1 % of its size."""
import numpy as np
import pytest
import torch

import oracle
import ptwm_b200
from ptwm_b200.compressor import CompressionConfig, HUFFMAN, IDENTITY, ORDER1_SCALE_AC, RANS, TANS, compress_model
from _data import mixed_model

pytestmark = pytest.mark.gpu

_TORCH = {oracle.DT_BF16: torch.bfloat16, oracle.DT_F16: torch.float16, oracle.DT_F32: torch.float32, oracle.DT_E4M3: torch.float8_e4m3fn,
          oracle.DT_U8: torch.uint8, oracle.DT_FP4X2: torch.uint8}


def to_cuda(specs):
    """specs -> ({name: cuda tensor}, usage map, specs as the device encoder sees them)"""
    tensors, usage, seen = {}, {}, []
    for s in specs:
        dt = _TORCH[s.dtype_code]
        t = torch.frombuffer(bytearray(s.raw), dtype=torch.uint8).view(dt).reshape(list(s.shape)) if s.raw else torch.empty(list(s.shape), dtype=dt)
        tensors[s.name] = t.cuda()
        spec = s
        if s.dtype_code == oracle.DT_FP4X2:  # carried as uint8 bytes on both sides; the fp4 chain still applies through `usage`
            spec = oracle.TensorSpec(s.name, oracle.DT_U8, s.shape, s.raw, usage="fp4")
        if spec.usage != "standard":
            usage[s.name] = spec.usage
        seen.append(spec)
    return tensors, usage, seen


@pytest.mark.parametrize("codec", [IDENTITY, HUFFMAN, RANS, TANS, ORDER1_SCALE_AC])
@pytest.mark.parametrize("chunk,crc,hash_", [(4096, True, False), (1000, False, True), (65536, True, True), (None, True, True)])
def test_forced_codec_bytes_equal_oracle(codec, chunk, crc, hash_):
    tensors, usage, specs = to_cuda(mixed_model())
    enc = compress_model(tensors, CompressionConfig(streaming_chunk=chunk, forced_codec=codec, emit_plane_crc=crc, emit_payload_hash=hash_), usage=usage)
    got = enc.to_bytes()
    want = oracle.write_container(specs, chunk_size=chunk, forced_codec=codec, emit_crc=crc, emit_hash=hash_)
    if got != want:
        first = next(i for i in range(min(len(got), len(want))) if got[i] != want[i])
        raise AssertionError(f"container differs at byte {first} (sizes {len(got)} / {len(want)})")


def test_selected_codecs_decode_in_oracle_and_match_size():
    tensors, usage, specs = to_cuda(mixed_model(2))
    full = (IDENTITY, HUFFMAN, RANS, TANS, ORDER1_SCALE_AC)
    for menu, chunk in ((IDENTITY, HUFFMAN, RANS), 8192), ((HUFFMAN, RANS), 8192), ((IDENTITY, HUFFMAN), 8192), (full, 8192), (full, None), ((IDENTITY, TANS), 3000):
        enc = compress_model(tensors, CompressionConfig(streaming_chunk=chunk, codec_menu=menu, emit_plane_crc=True), usage=usage)
        blob = enc.to_bytes()
        oc = oracle.Container(blob)
        for i, s in enumerate(specs):
            assert oc.decode(i) == s.raw, s.name
        theirs = []
        want = oracle.write_container(specs, chunk_size=chunk, menu=menu, emit_crc=True, choices=theirs)
        assert abs(len(blob) - len(want)) <= 0.01 * len(want), (menu, chunk, len(blob), len(want))
        if menu == full:  # the choice per plane is the oracle writer's (a restatement of the reference's trial encode)
            ours = [p for t in enc.plane_codecs.values() for p in t]
            differ = [(k, a, b) for k, (a, b) in enumerate(zip(ours, theirs)) if a != b]
            assert len(differ) <= 2, differ  # sizes within a few bytes of each other may fall either way (estimated here, trial-encoded there)
        # and the device decoder reads its own writer's output from device memory
        h = ptwm_b200.ContainerHandle(enc.to_tensor().cpu().numpy().tobytes(), device=0)
        for (name, t), s in zip(h.decode_model(), specs):
            assert t.contiguous().view(torch.uint8).cpu().numpy().tobytes() == s.raw, name


def test_encode_rejects_host_tensors_and_unknown_codec():
    with pytest.raises(ValueError):
        compress_model({"a": torch.zeros(4)})
    with pytest.raises(ValueError):
        compress_model({"a": torch.zeros(4, device="cuda")}, CompressionConfig(codec_menu=(4,)))  # zstd
    with pytest.raises(ptwm_b200.PtwmError):
        compress_model({"a": torch.zeros(4, device="cuda")}, CompressionConfig(forced_codec=4))


# ---- one plane through the reference's plane_codec ABI -------------------------------------
from test_gpu_decode import IDS, plane_cases  # noqa: E402  (canonical ids and the plane inputs of the decode tests)
from ptwm_b200 import _lib  # noqa: E402


NEEDED_UNTOUCHED = 0xDEADBEEF  # "On success *needed_out is left untouched" (flavor/native.rs:176-184 of the reference)


def encode_cuda(codec, plane: bytes, cap=None, state: bytes = b""):
    L = _lib.lib()
    src = torch.frombuffer(bytearray(plane or b"\0"), dtype=torch.uint8).cuda()
    cap = len(plane) + 16 if cap is None else cap
    out = torch.zeros(max(cap, 1), dtype=torch.uint8, device="cuda")
    needed = _lib.C.c_uint64(NEEDED_UNTOUCHED)
    rc = L.ptwm_plane_codec_v1_encode_cuda(1, _lib.C.create_string_buffer(state, len(state)) if state else None, len(state), bytes.fromhex(IDS[codec]), 32, src.data_ptr() if plane else 0, len(plane), out.data_ptr(), cap,
                                           _lib.C.byref(needed), 0)
    return rc, needed.value, bytes(out[:max(rc, 0)].cpu().numpy().tobytes())


@pytest.mark.parametrize("codec", [oracle.IDENTITY, oracle.HUFFMAN, oracle.RANS, oracle.TANS])
def test_plane_encode_cuda_matches_oracle(codec):
    coded = 0
    for name, plane in plane_cases():
        if len(plane) > (1 << 20):
            continue
        expect = oracle.plane_encode(codec, plane)[2]
        rc, needed, got = encode_cuda(codec, plane)
        assert rc == len(expect) and needed == NEEDED_UNTOUCHED, (name, rc, len(expect), needed)
        assert got == expect, name
        coded += codec != oracle.IDENTITY and got[:1] == b"\x01"
    if codec != oracle.IDENTITY:
        assert coded >= 5


def test_plane_encode_cuda_reports_the_size_it_needs():
    plane = bytes(range(256)) * 64
    rc, needed, _ = encode_cuda(oracle.RANS, plane, cap=8)
    assert rc == -2 and needed == len(oracle.plane_encode(oracle.RANS, plane)[2])
    rc, _, _ = encode_cuda(oracle.O1SAC, plane)  # no state to encode with: the flat ABI cannot hand a fitted one back
    assert rc == -5


def test_plane_encode_cuda_order1_scale_ac_with_a_given_state():
    """The shared-state form (codecs/order1_scale_ac.rs:620-633): the rows come from the caller, the payload is the range coder's bytes."""
    rng = np.random.default_rng(31)
    fit_on = (np.cumsum(rng.integers(-1, 2, (200, 128)), axis=1) + 100).astype(np.uint8).tobytes()
    state, sv, _ = oracle.plane_encode(oracle.O1SAC, fit_on, 128)
    for n in (1, 5, 4096, 70001):
        plane = (np.cumsum(rng.integers(-1, 2, n)) + 100).astype(np.uint8).tobytes()
        _, _, want = oracle.plane_encode(oracle.O1SAC, plane, 0, shared=state)
        rc, needed, got = encode_cuda(oracle.O1SAC, plane, state=state)
        assert rc == len(want) and got == want, (n, rc, len(want), _lib.last_error())
        assert oracle.plane_decode(oracle.O1SAC, got, n, state, sv) == plane
    rc, _, _ = encode_cuda(oracle.O1SAC, b"abc", state=state[:-1])
    assert rc == -1


def test_host_buffer_encode_round_trips_through_host_decode():
    L = _lib.lib()
    plane = np.random.default_rng(3).normal(0, 3, 50000).astype(np.int8).tobytes()
    out = _lib.C.create_string_buffer(len(plane) + 16)
    n = L.ptwm_plane_codec_v1_encode(plane, len(plane), out, len(plane) + 16)
    assert n > 0 and out.raw[:n] == oracle.plane_encode(oracle.RANS, plane)[2]
    back = _lib.C.create_string_buffer(len(plane))
    m = L.ptwm_plane_codec_v1_decode(out.raw[:n], n, back, len(plane))
    assert m == len(plane) and back.raw == plane


def test_scale_planes_go_to_order1_scale_ac_like_the_oracle_writer():
    """A block-scale tensor large enough for the context rows to pay for themselves: the full menu picks Order1ScaleAC for it
    on both sides, chunked and unchunked, and the sizes agree within 1 %."""
    from _data import specs_nvfp4, specs_mxfp4
    tensors, usage, specs = to_cuda(specs_nvfp4("nv", 1024, 2048, 41) + specs_mxfp4("mx", 1024, 4096, 42))
    for chunk in (65536, None):
        enc = compress_model(tensors, CompressionConfig(streaming_chunk=chunk, emit_plane_crc=True, emit_payload_hash=True), usage=usage)
        theirs = []
        want = oracle.write_container(specs, chunk_size=chunk, emit_crc=True, emit_hash=True, choices=theirs)
        ours = [p for t in enc.plane_codecs.values() for p in t]
        assert ours == theirs and ORDER1_SCALE_AC in ours, (chunk, ours, theirs)
        blob = enc.to_bytes()
        assert abs(len(blob) - len(want)) <= 0.01 * len(want), (chunk, len(blob), len(want))
        oc = oracle.Container(blob)
        for i, s in enumerate(specs):
            assert oc.decode(i) == s.raw, s.name
        h = ptwm_b200.ContainerHandle(blob, device=0)
        for (name, t), s in zip(h.decode_model(), specs):
            assert t.contiguous().view(torch.uint8).cpu().numpy().tobytes() == s.raw, name


def test_shared_scale_states_are_fitted_stored_once_and_used():
    """Passes 2 and 3 of the writer on unchunked planes: scale planes of two families get Order1ScaleAC states fitted over
    the whole model, the prelude stores the ones in use, the planes name them instead of carrying a state, the container is
    smaller than with a state per plane, and both decoders read it."""
    rng = np.random.default_rng(5)
    specs = []
    for k in range(6):  # two families of block scales over the same four values: one changes rarely along a row, one is noise
        rows, cols = 192 + 16 * k, 256
        if k % 2 == 0:
            vals = 120 + np.cumsum(rng.random((rows, cols)) < 0.06, axis=1) % 4
        else:
            vals = 120 + rng.integers(0, 4, (rows, cols))
        specs.append(oracle.TensorSpec(f"l{k}.scales", oracle.DT_U8, [rows, cols], vals.astype(np.uint8).tobytes(), usage="scale"))
    specs.append(oracle.TensorSpec("w.bf16", oracle.DT_BF16, [64, 512], (torch.randn(64, 512, generator=torch.Generator().manual_seed(3)) * 0.02).to(torch.bfloat16).view(torch.uint8).numpy().tobytes()))
    tensors, usage, specs = to_cuda(specs)
    base = compress_model(tensors, CompressionConfig(streaming_chunk=None, emit_plane_crc=True), usage=usage)
    enc = compress_model(tensors, CompressionConfig(streaming_chunk=None, emit_plane_crc=True, shared_states=True), usage=usage)
    blob = enc.to_bytes()
    assert b"order1_scale_ac/cluster_0_of_" in blob and b"order1_scale_ac/cluster_0_of_" not in base.to_bytes()
    assert enc.size < base.size, (enc.size, base.size)
    from ptwm_b200 import _lib
    host_states = _lib.fit_shared_states_host([sp.raw for sp in specs[:6]], [256] * 6)  # the same fit with the distances computed on the host
    assert len(host_states) == 2 and host_states[0] in blob
    assert b"_of_2" in blob  # two clusters describe the model in fewer bits than one; only states some plane uses are stored
    assert [enc.plane_codecs[f"l{k}.scales"] for k in (0, 2, 4)] == [[ORDER1_SCALE_AC]] * 3
    oc = oracle.Container(blob)
    for i, sp in enumerate(specs):
        assert oc.decode(i) == sp.raw, sp.name
    h = ptwm_b200.ContainerHandle(blob, device=0)
    for (name, t), sp in zip(h.decode_model(), specs):
        assert t.contiguous().view(torch.uint8).cpu().numpy().tobytes() == sp.raw, name
    # chunked planes carry their states inline whatever the option says
    a = compress_model(tensors, CompressionConfig(streaming_chunk=8192, shared_states=True), usage=usage).to_bytes()
    b = compress_model(tensors, CompressionConfig(streaming_chunk=8192), usage=usage).to_bytes()
    assert a == b


@pytest.mark.parametrize("seed", range(10))
def test_random_models_round_trip_through_both_decoders(seed):
    """Seeded random state dicts through the device encoder with random options (chunk size or whole planes, menu or a
    forced codec, candidate chains, integrity fields): the oracle and the device decoder both return the source bytes."""
    rng = np.random.default_rng(2000 + seed)
    tensors = {}
    for t in range(int(rng.integers(2, 6))):
        kind = ["bf16", "f16", "f32", "fp8", "u8", "bf16", "sparse_bf16"][int(rng.integers(0, 7))]
        rows, cols = int(rng.integers(1, 120)), int(rng.integers(1, 2500))
        g = torch.Generator().manual_seed(seed * 16 + t)
        w = torch.randn(rows, cols, generator=g) * 0.02
        if kind == "bf16":
            x = w.to(torch.bfloat16)
        elif kind == "sparse_bf16":  # low mantissa bits clear: what MantissaZeroStrip is for
            x = (w.to(torch.bfloat16).view(torch.int16) & ~0x7).view(torch.bfloat16)
        elif kind == "f16":
            x = w.to(torch.float16)
        elif kind == "f32":
            x = w
        elif kind == "fp8":
            x = (w / w.abs().amax() * 200).to(torch.float8_e4m3fn)
        else:
            x = ((torch.randn(rows * cols, generator=g) * 2.5).round().to(torch.int64) + 100).clamp(0, 255).to(torch.uint8)
        tensors[f"t{t}.{kind}"] = x.cuda()
    chunk = [None, 777, 4099, 8192, 32768, 65536][int(rng.integers(0, 6))]
    kw = dict(streaming_chunk=chunk, emit_plane_crc=bool(rng.integers(0, 2)), emit_payload_hash=bool(rng.integers(0, 2)))
    pick = int(rng.integers(0, 6))
    if pick < 4:
        kw["forced_codec"] = [IDENTITY, HUFFMAN, RANS, TANS][pick]
    elif pick == 4:
        kw["codec_menu"] = (IDENTITY, HUFFMAN, RANS, TANS)
    if pick >= 4 and rng.integers(0, 2):
        kw["candidate_chains"] = ("intdelta", "mzs")
    enc = compress_model(tensors, CompressionConfig(**kw))
    blob = enc.to_bytes()
    oc = oracle.Container(blob)
    h = ptwm_b200.ContainerHandle(blob, device=0)
    for i, ((name, got), (want_name, want)) in enumerate(zip(h.decode_model(), tensors.items())):
        raw = want.contiguous().view(torch.uint8).cpu().numpy().tobytes()
        assert name == want_name and got.contiguous().view(torch.uint8).cpu().numpy().tobytes() == raw, (name, kw)
        assert oc.decode(i) == raw, (name, kw)


# ---- chains with one more op between the split and a terminal --------------------------------------------
def _chain_model():
    """bf16 / fp16 / fp32 tensors for the candidate chains: `smooth` has slowly varying magnitudes (its exponent bytes differ
    little from one element to the next), `coarse` was rounded to few mantissa bits (every low mantissa byte ends in zero bits)."""
    rng = np.random.default_rng(51)
    n = 3 * 65536 + 777
    env = np.exp(np.cumsum(rng.normal(0, 0.02, n))) * 1e-3
    smooth = torch.from_numpy((env * rng.choice([-1.0, 1.0], n) * (1 + 0.3 * rng.random(n))).astype(np.float32))
    coarse16 = (torch.randn(n, generator=torch.Generator().manual_seed(52)) * 0.02).to(torch.bfloat16).view(torch.int16) & ~0x000F
    coarse32 = (torch.randn(n, generator=torch.Generator().manual_seed(53)) * 0.02).view(torch.int32) & ~0x0000003F
    plain = (torch.randn(n, generator=torch.Generator().manual_seed(54)) * 0.02).to(torch.bfloat16)
    return {"smooth.bf16": smooth.to(torch.bfloat16), "smooth.f32": smooth, "coarse.bf16": coarse16.view(torch.bfloat16), "coarse.f16": coarse16.view(torch.float16),
            "coarse.f32": coarse32.view(torch.float32), "plain.bf16": plain}


def _specs_of(tensors, post):
    code = {torch.bfloat16: oracle.DT_BF16, torch.float16: oracle.DT_F16, torch.float32: oracle.DT_F32}
    return [oracle.TensorSpec(n, code[t.dtype], list(t.shape), t.contiguous().view(torch.uint8).numpy().tobytes(), post=({p: op for p, op in [post[n]]} if n in post else None))
            for n, t in tensors.items()]


@pytest.mark.parametrize("chunk", [8192, None])
@pytest.mark.parametrize("codec", [None, RANS, TANS])
def test_given_chains_bytes_equal_oracle(chunk, codec):
    host = _chain_model()
    given = {"smooth.bf16": ("intdelta",), "smooth.f32": ("intdelta",), "coarse.bf16": ("mzs", 4), "coarse.f16": ("mzs", 2), "coarse.f32": ("mzs", 6)}
    planes = {"smooth.bf16": 1, "smooth.f32": 3, "coarse.bf16": 0, "coarse.f16": 0, "coarse.f32": 0}
    tensors = {n: t.cuda() for n, t in host.items()}
    cfg = CompressionConfig(streaming_chunk=chunk, forced_codec=codec, codec_menu=(IDENTITY, HUFFMAN, RANS), emit_plane_crc=True, emit_payload_hash=True)
    got = compress_model(tensors, cfg, post=given).to_bytes()
    specs = _specs_of(host, {n: (planes[n], op) for n, op in given.items()})
    want = oracle.write_container(specs, chunk_size=chunk, forced_codec=codec, menu=(IDENTITY, HUFFMAN, RANS), emit_crc=True, emit_hash=True)
    if codec is not None:
        assert got == want, next(i for i in range(min(len(got), len(want))) if got[i] != want[i])
    else:
        assert abs(len(got) - len(want)) <= 0.01 * len(want)
    oc = oracle.Container(got)
    for i, s in enumerate(specs):
        assert oc.decode(i) == s.raw, s.name
    h = ptwm_b200.ContainerHandle(got, device=0)
    for (name, t), s in zip(h.decode_model(), specs):
        assert t.contiguous().view(torch.uint8).cpu().numpy().tobytes() == s.raw, name
    with pytest.raises(ptwm_b200.PtwmError, match="non-zero low bits"):
        compress_model({"plain.bf16": tensors["plain.bf16"]}, cfg, post={"plain.bf16": ("mzs", 1)})


def test_candidate_chains_pick_what_the_oracle_writer_would():
    """Selection over {split, IntDelta, MantissaZeroStrip 1..4}: for every tensor the chain whose oracle-written container is the
    smallest (the first candidate on ties), which is how the reference's pass 1 chooses (compressor.rs:504-665)."""
    host = _chain_model()
    tensors = {n: t.cuda() for n, t in host.items()}
    cfg = CompressionConfig(streaming_chunk=16384, codec_menu=(IDENTITY, HUFFMAN, RANS), emit_plane_crc=True, candidate_chains=("intdelta", "mzs"))
    enc = compress_model(tensors, cfg)
    blob = enc.to_bytes()
    h = ptwm_b200.ContainerHandle(blob, device=0)
    for (name, t), src in zip(h.decode_model(), host.values()):
        assert t.contiguous().view(torch.uint8).cpu().numpy().tobytes() == src.contiguous().view(torch.uint8).numpy().tobytes(), name
    for name, t in host.items():
        last = 3 if t.dtype == torch.float32 else 1
        best, best_size = None, None
        for cand in [None, (last, ("intdelta",))] + [(0, ("mzs", k)) for k in (1, 2, 3, 4)]:
            try:
                size = len(oracle.write_container(_specs_of({name: t}, {name: cand} if cand else {}), chunk_size=16384, menu=(IDENTITY, HUFFMAN, RANS), emit_crc=True))
            except ValueError:
                continue  # the strip does not apply
            if best_size is None or size < best_size:
                best, best_size = cand, size
        one = compress_model({name: tensors[name]}, cfg)
        assert abs(one.size - best_size) <= 0.005 * best_size, (name, best, one.size, best_size)
    plain = compress_model(tensors, CompressionConfig(streaming_chunk=16384, codec_menu=(IDENTITY, HUFFMAN, RANS), emit_plane_crc=True)).size
    assert enc.size < 0.97 * plain  # the candidates pay on this data
