"""CPU oracle for the PTWM decode/encode hot path — TEST INFRASTRUCTURE.

ctypes front end over ``libptwm_oracle.so`` (the C++ restatement of ptwm-core's
coders, transforms, hashes and container reader in this folder) plus a small
container/frame writer in Python.  Only the test-suite, the smoke check and
the benchmark's CPU-baseline leg may import this package; the product
(``ptwm_b200``) never does.

Reference files restated (paths under ``crates/ptwm-core/src``): see the
headers of ``entropy.hpp``, ``codecs.hpp`` and ``container.hpp``; the writer
below follows ``ptwc.rs:76-93,160-226``, ``tensor_record_compact.rs:203-493``,
``chain/wire_compact.rs:140-245``, ``extension/compact_table.rs:123-158``,
``compressor.rs:316-381,996-1195`` and ``compact.rs:175-260``.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libptwm_oracle.so")

IDENTITY, HUFFMAN, RANS, ZSTD, TANS, O1SAC = 0, 1, 3, 4, 7, 0x11
PASS, M16, M32, FP8_E4M3, FP8_E5M2 = 0, 1, 2, 3, 4

# public dtype codes (dtype.rs:25-50)
DT_F32, DT_F16, DT_BF16, DT_U8, DT_I8, DT_E4M3, DT_E5M2, DT_FP4X2 = 1, 4, 6, 13, 17, 29, 30, 31
_CANON = {1: "float32", 2: "float", 4: "float16", 5: "half", 6: "bfloat16", 13: "uint8", 15: "uint32", 17: "int8",
          18: "int16", 19: "short", 20: "int32", 21: "int", 22: "int64", 23: "long", 24: "bool",
          29: "float8_e4m3fn", 30: "float8_e5m2", 31: "float4_e2m1fn_x2"}
_ELEM = {13: 1, 17: 1, 24: 1, 29: 1, 30: 1, 31: 1, 4: 2, 5: 2, 6: 2, 18: 2, 19: 2, 1: 4, 2: 4, 15: 4, 20: 4, 21: 4, 22: 8, 23: 8}
_CHAIN_DT = {1: 0x0003, 2: 0x0003, 4: 0x0002, 5: 0x0002, 6: 0x000F, 13: 0x0006, 15: 0x000A, 17: 0x0005, 18: 0x0007, 19: 0x0007,
             20: 0x0009, 21: 0x0009, 22: 0x000B, 23: 0x000B, 29: 0x0010, 30: 0x0011, 31: 0x001F}


def build(force: bool = False) -> str:
    """Compile the shared library with the committed Makefile (g++)."""
    srcs = [os.path.join(_HERE, f) for f in ("capi.cpp", "entropy.hpp", "codecs.hpp", "container.hpp")]
    if force or not os.path.exists(_LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs):
        subprocess.run(["make", "-C", _HERE, "CXX=g++"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_last_error.restype = C.c_char_p
        L.oracle_crc32.restype = C.c_uint32
        L.oracle_crc32.argtypes = [C.c_char_p, C.c_size_t]
        L.oracle_xxh64.restype = C.c_uint64
        L.oracle_xxh64.argtypes = [C.c_char_p, C.c_size_t, C.c_uint64]
        L.oracle_free.argtypes = [C.c_void_p]
        L.oracle_container_open.restype = C.c_void_p
        L.oracle_container_open.argtypes = [C.c_void_p, C.c_size_t]
        L.oracle_container_close.argtypes = [C.c_void_p]
        L.oracle_container_count.restype = C.c_size_t
        L.oracle_container_count.argtypes = [C.c_void_p]
        _lib = L
    return _lib


class OracleError(RuntimeError):
    pass


def _check(rc):
    if rc != 0:
        raise OracleError(lib().oracle_last_error().decode("utf-8", "replace"))


def _take(ptr, n) -> bytes:
    data = C.string_at(ptr, n.value) if n.value else b""
    lib().oracle_free(ptr)
    return data


def crc32(data: bytes) -> int:
    return lib().oracle_crc32(bytes(data), len(data))


def xxh64(data: bytes, seed: int = 0) -> int:
    return lib().oracle_xxh64(bytes(data), len(data), seed)


def plane_encode(codec: int, plane: bytes, row_len: int = 0, shared: Optional[bytes] = None):
    """PlaneCodec::encode → (state_bytes, state_version, payload)."""
    st, pl = C.c_void_p(), C.c_void_p()
    sl, pll = C.c_size_t(), C.c_size_t()
    sv = C.c_uint8()
    _check(lib().oracle_plane_encode(C.c_int(codec), bytes(plane), C.c_size_t(len(plane)), C.c_size_t(row_len),
                                     shared if shared is not None else None, C.c_size_t(len(shared) if shared else 0),
                                     C.byref(st), C.byref(sl), C.byref(sv), C.byref(pl), C.byref(pll)))
    return _take(st, sl), sv.value, _take(pl, pll)


def plane_decode(codec: int, payload: bytes, decoded_len: int, state: bytes = b"", state_version: int = 0,
                 row_len: int = 0, max_len: Optional[int] = None) -> bytes:
    """PlaneCodec::decode_bounded."""
    out, ol = C.c_void_p(), C.c_size_t()
    _check(lib().oracle_plane_decode(C.c_int(codec), C.c_uint8(state_version), bytes(state), C.c_size_t(len(state)), bytes(payload),
                                     C.c_size_t(len(payload)), C.c_size_t(row_len), C.c_size_t(decoded_len),
                                     C.c_size_t(decoded_len if max_len is None else max_len), C.byref(out), C.byref(ol)))
    return _take(out, ol)


def raw_compress(codec: int, data: bytes) -> bytes:
    """entropy::{huffman,rans,tans}::compress; b'' means "store raw"."""
    out, ol = C.c_void_p(), C.c_size_t()
    _check(lib().oracle_raw_compress(C.c_int(codec), bytes(data), C.c_size_t(len(data)), C.byref(out), C.byref(ol)))
    return _take(out, ol)


def raw_decompress(codec: int, blob: bytes, n: int) -> bytes:
    dst = C.create_string_buffer(max(n, 1))
    _check(lib().oracle_raw_decompress(C.c_int(codec), bytes(blob), C.c_size_t(len(blob)), dst, C.c_size_t(n)))
    return dst.raw[:n]


def split_forward(kind: int, raw: bytes) -> list[bytes]:
    out, pl = C.c_void_p(), C.c_size_t()
    _check(lib().oracle_split_forward(C.c_int(kind), bytes(raw), C.c_size_t(len(raw)), C.byref(out), C.byref(pl)))
    n = {PASS: 1, M32: 4}.get(kind, 2)
    tot = C.c_size_t(pl.value * n)
    data = _take(out, tot)
    return [data[i * pl.value:(i + 1) * pl.value] for i in range(n)]


def merge_inverse(kind: int, planes: Sequence[bytes]) -> bytes:
    out, ol = C.c_void_p(), C.c_size_t()
    blob = b"".join(planes)
    _check(lib().oracle_merge_inverse(C.c_int(kind), blob, C.c_size_t(len(planes[0])), C.byref(out), C.byref(ol)))
    return _take(out, ol)


def quantize_pmf(raw: Sequence[int], total: int) -> list[int]:
    n = len(raw)
    a = (C.c_uint32 * n)(*raw)
    o = (C.c_uint16 * n)()
    lib().oracle_quantize_pmf(a, C.c_size_t(n), C.c_uint32(total), o)
    return list(o)


def install_zstd(path: str = "libzstd.so.1") -> bool:
    """Test-only: decode the Zstd planes of the reference's golden fixtures
    through the system libzstd.  Zstd is outside the hot path."""
    return lib().oracle_install_zstd(path.encode()) == 0


def num_procs() -> int:
    return lib().oracle_num_procs()


class Container:
    """ContainerReader over a \\x89PTWC blob (container.rs:1395-1789)."""

    def __init__(self, blob):
        self._buf = (C.c_char * len(blob)).from_buffer_copy(blob) if not isinstance(blob, C.Array) else blob
        self._h = lib().oracle_container_open(C.addressof(self._buf), len(blob))
        if not self._h:
            raise OracleError(lib().oracle_last_error().decode("utf-8", "replace"))
        out, ol = C.c_void_p(), C.c_size_t()
        _check(lib().oracle_container_describe(C.c_void_p(self._h), C.byref(out), C.byref(ol)))
        self.tensors = json.loads(_take(out, ol))["tensors"]
        self.names = [t["name"] for t in self.tensors]

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oracle_container_close(C.c_void_p(self._h))
            self._h = None

    def decode(self, index_or_name, verify: bool = True) -> bytes:
        i = self.names.index(index_or_name) if isinstance(index_or_name, str) else index_or_name
        n = self.tensors[i]["orig_size"]
        dst = C.create_string_buffer(max(n, 1))
        _check(lib().oracle_container_decode_tensor(C.c_void_p(self._h), C.c_size_t(i), C.c_int(verify), dst, C.c_size_t(n)))
        return dst.raw[:n]

    def decode_range(self, first: int, count: int, threads: int = 0, verify: bool = True, keep: bool = False):
        """decode_model over a tensor range → (decoded_bytes, seconds[, data])."""
        offs, total = [], 0
        for t in self.tensors[first:first + count]:
            offs.append(total)
            total += t["orig_size"]
        dst = C.create_string_buffer(max(total, 1)) if keep else None
        oa = (C.c_uint64 * max(count, 1))(*offs)
        dec, sec = C.c_uint64(), C.c_double()
        _check(lib().oracle_container_decode_range(C.c_void_p(self._h), C.c_size_t(first), C.c_size_t(count), C.c_int(threads), C.c_int(verify),
                                                   dst, oa, C.byref(dec), C.byref(sec)))
        if keep:
            return dec.value, sec.value, dst.raw[:total]
        return dec.value, sec.value


def decode_compact(blob: bytes):
    """decode_compact (compact.rs:407-457) → (raw, description dict)."""
    raw, rl, d, dl = C.c_void_p(), C.c_size_t(), C.c_void_p(), C.c_size_t()
    _check(lib().oracle_decode_compact(bytes(blob), C.c_size_t(len(blob)), C.byref(raw), C.byref(rl), C.byref(d), C.byref(dl)))
    return _take(raw, rl), json.loads(_take(d, dl))


# ---------------------------------------------------------------------------
# Writer (Python; test-side only)
# ---------------------------------------------------------------------------
def varint(v: int) -> bytes:
    out = bytearray()
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


# Compact terminal role bytes (chain/wire_compact.rs:434-459)
ROLE_SCALE_E8M0, ROLE_SCALE_E4M3, ROLE_GLOBAL_F32 = 0x00, 0x01, 0x08 + 3
ROLE_NIB_EXP, ROLE_NIB_SM, ROLE_FP4, ROLE_EXP = 0x10, 0x11, 0x18, 0x19
ROLE_INT8 = 0xC0 + 8 - 1


def role_mantissa(i, of):
    return 0x40 + 8 * (of - 1) + i


# Op wire ids (transforms/op.rs:11-36)
OP_SOURCE, OP_R16, OP_R32, OP_RE4M3, OP_RE5M2, OP_BSPLIT, OP_NSPLIT, OP_PASS = 0, 0x10, 0x11, 0x12, 0x13, 0x20, 0x21, 0x30
OP_INTDELTA, OP_MZS = 0x52, 0x64

# Record role byte per terminal role (compressor.rs:124-147)
_PLANE_ROLE = {ROLE_SCALE_E8M0: 2, ROLE_SCALE_E4M3: 2, ROLE_GLOBAL_F32: 2, ROLE_NIB_EXP: 3, ROLE_NIB_SM: 4, ROLE_FP4: 1, ROLE_EXP: 3, ROLE_INT8: 1}


def _plane_role(code: int) -> int:
    if 0x40 <= code < 0x80:
        return 5
    return _PLANE_ROLE[code]


@dataclass
class TensorSpec:
    """One tensor to write.  ``usage`` picks the production chain
    (python/ptwm/preprocessing/_chains.py:320-357,610-727): 'standard',
    'scale' (E4M3 / E8M0 block scales), 'global_scale' (fp32), 'fp4'."""
    name: str
    dtype_code: int
    shape: Sequence[int]
    raw: bytes
    usage: str = "standard"
    input_format: int = 2  # Format.TORCH (python/ptwm/_config.py)
    # per-plane op between a byte split and its terminal, {plane: ("intdelta",) | ("mzs", k)}
    # (python/ptwm/preprocessing/_chains.py:360-389,486-560)
    post: Optional[dict] = None


def source_params(shape, chain_dtype) -> bytes:
    return bytes([len(shape)]) + b"".join(int(d).to_bytes(4, "little") for d in shape) + int(chain_dtype).to_bytes(2, "little")


def chain_for(spec: TensorSpec):
    """→ (kind, nodes [(op, params)], terminal roles)."""
    dt, sh = spec.dtype_code, list(spec.shape)
    if spec.usage == "scale":
        if dt == DT_E4M3:
            return PASS, [(OP_SOURCE, source_params(sh, 0x0010)), (OP_PASS, b"")], [ROLE_SCALE_E4M3]
        if dt == DT_U8:
            return PASS, [(OP_SOURCE, source_params(sh, 0x0006)), (OP_PASS, b"")], [ROLE_SCALE_E8M0]
        raise ValueError("scale usage needs float8_e4m3fn or uint8")
    if spec.usage == "global_scale":
        return PASS, [(OP_SOURCE, source_params(sh, 0x0003)), (OP_PASS, b"")], [ROLE_GLOBAL_F32]
    if spec.usage == "fp4" or dt == DT_FP4X2:
        return PASS, [(OP_SOURCE, source_params(sh, 0x001F)), (OP_PASS, b"")], [ROLE_FP4]
    if dt in (DT_BF16, DT_F16):  # fp16 uses the bf16-named chain (Source dtype 0x000F): _chains.py:326,1163-1165
        return M16, [(OP_SOURCE, source_params(sh, 0x000F)), (OP_R16, b""), (OP_BSPLIT, b"\x02")], [role_mantissa(0, 2), ROLE_EXP]
    if dt == DT_F32:
        return M32, [(OP_SOURCE, source_params(sh, 0x0003)), (OP_R32, b""), (OP_BSPLIT, b"\x04")], [role_mantissa(i, 4) for i in range(3)] + [ROLE_EXP]
    if dt == DT_E4M3:
        return FP8_E4M3, [(OP_SOURCE, source_params(sh, 0x0010)), (OP_RE4M3, b""), (OP_NSPLIT, b"")], [ROLE_NIB_EXP, ROLE_NIB_SM]
    if dt == DT_E5M2:
        return FP8_E5M2, [(OP_SOURCE, source_params(sh, 0x0011)), (OP_RE5M2, b""), (OP_NSPLIT, b"")], [ROLE_NIB_EXP, ROLE_NIB_SM]
    if dt in (DT_U8, DT_I8):
        return PASS, [(OP_SOURCE, source_params(sh, _CHAIN_DT[dt])), (OP_PASS, b"")], [ROLE_INT8]
    raise ValueError(f"no production chain for dtype code {dt}")


def bound_params(shape, dtype_code) -> Optional[bytes]:
    cd = _CHAIN_DT.get(dtype_code)
    if cd is None or len(shape) > 255 or any(d > 0xFFFFFFFF for d in shape):
        return None
    return source_params(shape, cd)


def chain_graph(spec: TensorSpec):
    """chain_for plus the spec's per-plane ops -> (kind, nodes, edges [(src, out, dst, in)], terminals [(node, out, role)])."""
    kind, nodes, roles = chain_for(spec)
    nodes = list(nodes)
    edges = [(i, 0, i + 1, 0) for i in range(len(nodes) - 1)]
    terms = [(len(nodes) - 1, i, role) for i, role in enumerate(roles)]
    for plane in sorted(spec.post or {}):
        op = spec.post[plane]
        if kind not in (M16, M32) or not 0 <= plane < len(roles):
            raise ValueError("per-plane ops go on the planes of a byte split")
        nodes.append((OP_INTDELTA, b"") if op[0] == "intdelta" else (OP_MZS, bytes([op[1]])))
        edges.append((2, plane, len(nodes) - 1, 0))
        terms[plane] = (len(nodes) - 1, 0, roles[plane])
    return kind, nodes, edges, terms


def post_forward(spec: TensorSpec, plane_index: int, plane: bytes) -> bytes:
    """transforms/int_delta.rs:36-44 (byte width) and transforms/mantissa_zero.rs forward on one terminal plane."""
    op = (spec.post or {}).get(plane_index)
    if op is None:
        return plane
    import numpy as np
    a = np.frombuffer(plane, dtype=np.uint8)
    if op[0] == "intdelta":
        return np.diff(a, prepend=np.uint8(0)).astype(np.uint8).tobytes()
    k = int(op[1])
    if (a & ((1 << k) - 1)).any():
        raise ValueError("MantissaZeroStrip: plane has a byte with non-zero low bits")
    return (a >> k).astype(np.uint8).tobytes()


def write_cw2(nodes, terms, edges, bound: Optional[bytes], deferred: bool, op_ref) -> bytes:
    """chain/wire_compact.rs:140-245: leading edges of the form (i, 0) -> (i + 1, 0) are the spine and only counted."""
    out = bytearray(varint(len(nodes)) + varint(len(edges)) + varint(len(terms)))
    for op, params in nodes:
        out += varint(op_ref(op))
        if op == OP_SOURCE and ((deferred and params == b"") or (not deferred and bound is not None and params == bound)):
            out += varint(0)
            continue
        out += varint(len(params)) + params
    if edges:
        spine = 0
        while spine < len(edges) and tuple(edges[spine]) == (spine, 0, spine + 1, 0):
            spine += 1
        out += varint(spine)
        for e in edges[spine:]:
            out += b"".join(varint(v) for v in e) + b"\x00"
    for node, o, role in terms:
        out += bytes([(node << 4) | o, role])
    return bytes(out)


_CODEC_ORDER = [IDENTITY, HUFFMAN, RANS, ZSTD, 5, 6, TANS, O1SAC]  # extension/builtins.rs:35-52


def encode_plane_chunked(codec: int, plane: bytes, chunk_size: int):
    """compressor.rs:316-381 → (payload, [(offset, decoded_size)])."""
    chunk_size = max(int(chunk_size), 1)
    payload, entries = bytearray(), []
    pieces = [plane[i:i + chunk_size] for i in range(0, len(plane), chunk_size)] or [b""]
    for piece in pieces:
        st, sv, pl = plane_encode(codec, piece, 0)
        entries.append((len(payload), len(piece)))
        payload += bytes([sv]) + len(st).to_bytes(4, "little") + st + pl
    return bytes(payload), entries


def select_codec(plane: bytes, menu: Sequence[int], row_len: int, role: int):
    """Trial-encode (select.rs:27-64 over the dispatch order of
    dispatch.rs:13-49): smallest state+payload wins, first on ties."""
    order = []
    scale_role = role in (ROLE_SCALE_E8M0, ROLE_SCALE_E4M3, 0x02) or 0x08 <= role <= 0x0C
    if O1SAC in menu and scale_role and role in (ROLE_SCALE_E8M0, ROLE_SCALE_E4M3, 0x02, 0x08, 0x09, 0x0A) and row_len:
        order.append(O1SAC)
    order += [c for c in (HUFFMAN, RANS, TANS) if c in menu]
    if IDENTITY in menu:
        order.append(IDENTITY)
    best = None
    for c in order:
        st, sv, pl = plane_encode(c, plane, row_len if c == O1SAC else 0)
        size = len(st) + len(pl)
        if best is None or size < best[0]:
            best = (size, c, st, sv, pl)
    if best is None:
        raise ValueError("empty codec menu")
    return best[1:]


def write_container(specs: Sequence[TensorSpec], *, chunk_size: Optional[int] = None, menu: Sequence[int] = (IDENTITY, HUFFMAN, RANS, TANS, O1SAC),
                    forced_codec: Optional[int] = None, emit_hash: bool = False, emit_crc: bool = False, choices: Optional[list] = None) -> bytes:
    """compress_model (compressor.rs:972-1200) with one candidate chain per
    tensor and no shared-state pass, compact layout.  `choices`, when given, receives
    the codec picked for every plane in container order."""
    plans = []
    registry: list = []  # [(nodes, roles)] after binding
    for s in specs:
        kind, nodes, edges, terms = chain_graph(s)
        roles = [t[2] for t in terms]
        if len(s.raw) != int.__mul__(_ELEM[s.dtype_code], _prod(s.shape)):
            raise ValueError(f"{s.name}: raw length does not match shape × dtype")
        bp = bound_params(s.shape, s.dtype_code)
        if bp is not None and nodes[0][1] == bp:
            nodes = [(OP_SOURCE, b"")] + nodes[1:]
        key = (tuple(nodes), tuple(edges), tuple(terms))
        if key not in registry:
            registry.append(key)
        planes = [post_forward(s, i, p) for i, p in enumerate(split_forward(kind, s.raw))]
        src_row = s.shape[-1] if len(s.shape) else 0
        chosen = []
        for plane, role in zip(planes, roles):
            row_len = src_row if kind == PASS else 0  # split ops emit Flat planes (transforms/byte_split.rs:76)
            if forced_codec is not None:
                st, sv, pl = plane_encode(forced_codec, plane, row_len if forced_codec == O1SAC else 0)
                chosen.append((forced_codec, st, sv, pl, row_len))
            else:
                c, st, sv, pl = select_codec(plane, menu, row_len, role)
                chosen.append((c, st, sv, pl, row_len))
        if choices is not None:
            choices.extend(c[0] for c in chosen)
        plans.append((s, kind, registry.index(key), roles, planes, chosen))

    # Extension Table: chain ops in registry order, then the used codecs in built-in order (container.rs:167-223).
    table: list = []
    for nodes, _e, _t in registry:
        for op, _p in nodes:
            if (1, op) not in table:
                table.append((1, op))
    used = {c for p in plans for (c, *_rest) in p[5]}
    for c in _CODEC_ORDER:
        if c in used:
            table.append((2, c))
    et = bytearray(varint(len(table)))
    for tag, wid in table:
        et += bytes([tag]) + varint(wid)
    prelude = (0).to_bytes(4, "little")
    reg = bytearray(varint(len(registry)))
    for nodes, edges, terms in registry:
        cb = write_cw2(list(nodes), list(terms), list(edges), None, True, lambda op: table.index((1, op)))
        reg += varint(len(cb)) + cb

    body, index = bytearray(), bytearray(varint(len(plans)))
    for s, kind, chain_id, roles, planes, chosen in plans:
        rec = bytearray()
        tflags = 0x08 | (0x01 if emit_hash else 0)
        rec.append(tflags)
        rec += varint(chain_id) + varint(s.dtype_code) + bytes([s.input_format]) + varint(len(s.raw))
        rec += varint(len(s.shape)) + b"".join(varint(int(d)) for d in s.shape)
        if emit_hash:
            rec += xxh64(s.raw).to_bytes(8, "little")
        rec += varint(len(planes))
        for plane, role, (codec, st, sv, pl, row_len) in zip(planes, roles, chosen):
            if chunk_size is not None:
                payload, entries = encode_plane_chunked(codec, plane, chunk_size)
                state_source, st, sv, row_len = 0, b"", 0, 0
            else:
                payload, entries = pl, None
                state_source = 0 if codec == IDENTITY else 1  # menu items other than Identity are Inline (compressor.rs:204-212)
                if codec != O1SAC:
                    row_len = row_len  # record layout = plane layout (compressor.rs:1117-1121)
            pflags = (state_source << 2) | (0x01 if emit_crc else 0) | (0x02 if entries is not None else 0) | (0x10 if row_len else 0)
            extra = sv != 0
            if extra:
                pflags |= 0x20
            rec += bytes([pflags, _plane_role(role)]) + varint(table.index((2, codec)))
            if extra:
                rec += bytes([sv]) + varint(0)
            if state_source == 1:
                rec += varint(len(st))
            rec += varint(len(payload))
            if row_len:
                rec += varint(row_len)
            if emit_crc:
                rec += crc32(plane).to_bytes(4, "little")
            if entries is not None:
                rec += varint(len(entries)) + b"".join(varint(o) + varint(d) for o, d in entries)
            rec += st + payload
        nb = s.name.encode()
        index += varint(len(nb)) + nb + varint(len(rec))
        body += rec

    header = bytearray(b"\x89PTWC\r\n\x1a\n" + b"\x00\x00" + varint(len(et)) + varint(len(prelude)) + varint(len(reg)))
    header += xxh64(bytes(header) + bytes(et) + prelude + bytes(reg)).to_bytes(8, "little")
    return bytes(header) + bytes(et) + prelude + bytes(reg) + bytes(body) + bytes(index) + len(index).to_bytes(8, "little") + b"\x89TWMEOF\x1a"


def _prod(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


def write_compact(spec: TensorSpec, *, menu: Sequence[int] = (IDENTITY, HUFFMAN, RANS, TANS, O1SAC), forced_codec: Optional[int] = None,
                  emit_hash: bool = False, emit_crc: bool = False) -> bytes:
    """compress_compact (compact.rs:175-312): one tensor as a \\x89PTWS frame."""
    kind, nodes, edges, terms = chain_graph(spec)
    roles = [t[2] for t in terms]
    raw = spec.raw
    out = bytearray(b"\x89PTWS")
    flags = 0x04
    hdr = varint(spec.dtype_code) + bytes([spec.input_format])
    hdr += varint(len(spec.shape)) + b"".join(varint(int(d)) for d in spec.shape)
    if emit_hash:
        flags |= 0x01
        hdr += xxh64(raw).to_bytes(8, "little")
    plane_crc = emit_crc and not emit_hash
    bp = bound_params(spec.shape, spec.dtype_code)
    body = bytearray(write_cw2(nodes, terms, edges, bp, False, lambda op: op))
    src_row = spec.shape[-1] if len(spec.shape) else 0
    for plane, role in zip([post_forward(spec, i, p) for i, p in enumerate(split_forward(kind, raw))], roles):
        row_len = src_row if kind == PASS else 0
        if forced_codec is not None:
            codec = forced_codec
            st, sv, pl = plane_encode(codec, plane, row_len if codec == O1SAC else 0)
        else:
            codec, st, sv, pl = select_codec(plane, menu, row_len, role)
        if codec == IDENTITY:
            body += varint(codec << 2 | 0)
        elif sv == 0 and not st:
            body += varint(codec << 2 | 2)
        else:
            body += varint(codec << 2 | 1) + bytes([sv]) + varint(len(st)) + st
        body += varint(len(pl))
        if plane_crc:
            body += crc32(plane).to_bytes(4, "little")
        body += pl
    if len(body) < len(raw):
        if plane_crc:
            flags |= 0x02
        payload = bytes(body)
    else:
        flags |= 0x20
        payload = raw
    out.append(flags)
    return bytes(out) + hdr + payload
