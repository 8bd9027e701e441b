"""A walker over the legacy ``\\x89PTWM`` layout, for tests only: just enough to
find a tensor's planes (docs/architecture/wire-format.md:101-347 of the
reference; header.rs, prelude.rs, tensor_record.rs:276-440,
plane_record.rs:118-260, index.rs:29-70)."""
import struct


def shared_states(blob: bytes) -> dict:
    pre_off = struct.unpack_from("<Q", blob, 75)[0]
    pos = pre_off
    count = struct.unpack_from("<I", blob, pos)[0]
    pos += 4
    out = {}
    for _ in range(count):
        sid, codec, version, mask = struct.unpack_from("<HHBB", blob, pos)
        nl = struct.unpack_from("<H", blob, pos + 16)[0]
        pos += 18 + nl + (4 - nl % 4) % 4
        sl = struct.unpack_from("<I", blob, pos)[0]
        pos += 4
        out[sid] = dict(codec=codec, version=version, state=blob[pos:pos + sl])
        pos += sl
    return out


def tensors(blob: bytes) -> dict:
    """{name: dict(orig_size, planes=[dict(codec, state_source, state_version, state_info, row_len, inline_state, payload, chunks)])}
    for records without an inline chain or dependencies."""
    idx_off = struct.unpack_from("<Q", blob, 59)[0]
    count = struct.unpack_from("<Q", blob, idx_off)[0]
    out = {}
    for i in range(count):
        _, off, _ = struct.unpack_from("<QQQ", blob, idx_off + 8 + 24 * i)
        chain_ref, dtype, _fmt, nplanes, flags, _res, orig = struct.unpack_from("<HHBBBBQ", blob, off)
        nl = struct.unpack_from("<H", blob, off + 16)[0]
        name = blob[off + 18:off + 18 + nl].decode()
        pos = off + 18 + nl + (4 - nl % 4) % 4
        if chain_ref & 0x8000 or flags & 0x01:
            continue
        if flags & 0x04:
            pos += 8
        if flags & 0x02:
            pos += 4 + struct.unpack_from("<I", blob, pos)[0]
        planes = []
        for _ in range(nplanes):
            _role, pf, codec, _tidx, ssrc, sver, sinfo, inline_len, payload_len = struct.unpack_from("<BBHHBBHIQ", blob, pos)
            pos += 22
            if pf & 0x02:
                pos += 4
            chunks = None
            if pf & 0x01:
                n = struct.unpack_from("<I", blob, pos)[0]
                pos += 4
                chunks = [struct.unpack_from("<II", blob, pos + 8 * k) for k in range(n)]
                pos += 8 * n
            assert ssrc != 3
            layout = blob[pos]
            pos += 1
            row_len = 0
            if layout == 1:
                row_len = struct.unpack_from("<I", blob, pos)[0]
                pos += 4
            inline_state = blob[pos:pos + inline_len]
            pos += inline_len
            payload = blob[pos:pos + payload_len]
            pos += payload_len
            planes.append(dict(codec=codec, state_source=ssrc, state_version=sver, state_info=sinfo, row_len=row_len, inline_state=inline_state,
                               payload=payload, chunks=chunks))
        out[name] = dict(orig_size=orig, dtype=dtype, planes=planes)
    return out
