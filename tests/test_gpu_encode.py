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
