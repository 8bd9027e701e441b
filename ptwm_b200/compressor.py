"""Encode on CUDA: tensors in device memory to a compact ``\\x89PTWC`` container.

Host-side mirror of the reference's model writer (``_rust.compress_model``,
crates/ptwm-py/src/lib.rs:348-508; ``compress_safetensors_file`` options in
python/ptwm/integrations/_compress_safetensors.py:182-423): explicit chains
(the plain split / passthrough set), a codec menu or a forced codec, chunked
planes, optional plane CRC-32 and XXH64 payload hash.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Mapping, Optional, Sequence

import torch

from . import _lib
from .container import PtwmError, _check, stream_handle

IDENTITY, HUFFMAN, RANS, TANS, ORDER1_SCALE_AC = 0, 1, 3, 7, 0x11
_MENU_BIT = {IDENTITY: 1, HUFFMAN: 2, RANS: 4, TANS: 8, ORDER1_SCALE_AC: 16}
_CHUNK_NONE = 0xFFFFFFFF
_USAGE = {"standard": 0, "scale": 1, "global_scale": 2, "fp4": 3}

_DTYPE_CODES = {torch.float32: 1, torch.float16: 4, torch.bfloat16: 6, torch.uint8: 13, torch.int8: 17, torch.float8_e4m3fn: 29, torch.float8_e5m2: 30}
if hasattr(torch, "float4_e2m1fn_x2"):
    _DTYPE_CODES[torch.float4_e2m1fn_x2] = 31


@dataclass(frozen=True, kw_only=True)
class CompressionConfig:
    """``streaming_chunk`` = plane bytes per chunk (CompressorOptions.chunk_size),
    ``None`` = unchunked planes, the reference's default (a plane is then four
    serial streams, or one: slow to write and to read on a GPU);
    ``codec_menu`` = codec wire ids selection may use (Order1ScaleAC is only ever
    offered to scale planes with a row layout); ``forced_codec`` = one codec for
    every plane (the reference's method_hint fast path);
    ``emit_plane_crc`` / ``emit_payload_hash`` as in python/ptwm/_config.py:177-184."""
    streaming_chunk: Optional[int] = 65536
    codec_menu: Sequence[int] = (IDENTITY, HUFFMAN, RANS, TANS, ORDER1_SCALE_AC)
    # Candidate chains tried beside the plain split for every 16- / 32-bit float tensor ("intdelta": IntDelta on the
    # exponent plane; "mzs": MantissaZeroStrip(1..4) on mantissa plane 0); the smallest total wins, the plain split on ties
    # (the reference's STANDARD candidate lists, python/ptwm/preprocessing/_chains.py:1151-1185, as far as the decoder goes).
    candidate_chains: Sequence[str] = ()
    # The writer's passes 2 and 3 (compressor.rs:834-939): Order1ScaleAC states fitted over all scale planes of the model
    # (clustered, the cluster count chosen by description length), stored once in the container's prelude, and used by
    # every scale plane whose payload comes out smaller that way.  Whole planes only (streaming_chunk=None) and only when
    # the codec is chosen from the menu; ignored otherwise, as in the reference.
    shared_states: bool = False
    forced_codec: Optional[int] = None
    emit_plane_crc: bool = False
    emit_payload_hash: bool = False


class EncodedContainer:
    """A container held in device memory by the library."""

    def __init__(self, handle, names: list[str], n_planes: list[int], device: int):
        self._e = handle
        self.names = names
        self.device = device
        L = _lib.lib()
        self.size = L.ptwm_b200_encoded_size(handle)
        self.plane_codecs = {n: [L.ptwm_b200_encoded_plane_codec(handle, i, p) for p in range(k)] for i, (n, k) in enumerate(zip(names, n_planes))}

    def __del__(self):
        if getattr(self, "_e", None):
            _lib.lib().ptwm_b200_encoded_free(self._e)
            self._e = None

    def to_bytes(self) -> bytes:
        buf = C.create_string_buffer(max(self.size, 1))
        _check(_lib.lib().ptwm_b200_encoded_copy(self._e, buf, self.size))
        return buf.raw[:self.size]

    def to_tensor(self) -> torch.Tensor:
        """The container bytes as a CUDA uint8 tensor (a copy owned by torch)."""
        t = torch.empty(self.size, dtype=torch.uint8, device=torch.device("cuda", self.device))
        if self.size:
            _check(_lib.lib().ptwm_b200_encoded_copy_to_device(self._e, t.data_ptr(), t.numel(), stream_handle(self.device)))
        return t


def _planes_of(code: int, usage: int) -> int:
    if usage != 0 or code in (13, 17, 31):
        return 1
    return 4 if code == 1 else 2


def compress_model(tensors: Mapping[str, torch.Tensor], config: Optional[CompressionConfig] = None, *, usage: Optional[Mapping[str, str]] = None,
                   device: Optional[int] = None, post: Optional[Mapping[str, tuple]] = None) -> EncodedContainer:
    """Encode CUDA tensors into one container.  ``usage`` maps a tensor name to
    'scale', 'global_scale' or 'fp4' for the microscaling chains; everything
    else gets the standard chain of its dtype.  ``post`` fixes the chain of a
    16- / 32-bit float tensor instead of leaving it to ``candidate_chains``:
    ``("intdelta",)`` or ``("mzs", k)``."""
    cfg = config or CompressionConfig()
    usage = usage or {}
    post = post or {}
    names = list(tensors)
    arr = (_lib.EncodeTensor * max(len(names), 1))()
    keep = []
    n_planes = []
    dev = device
    for i, name in enumerate(names):
        t = tensors[name]
        if not t.is_cuda:
            raise ValueError(f"{name}: compress_model reads tensors from device memory; move it to CUDA first")
        dev = t.device.index if dev is None else dev
        if t.device.index != dev:
            raise ValueError(f"{name}: tensors live on different devices")
        code = _DTYPE_CODES.get(t.dtype)
        if code is None:
            raise TypeError(f"{name}: no dtype code for {t.dtype}")
        t = t.contiguous()
        keep.append(t)
        u = _USAGE[usage.get(name, "standard")]
        e = arr[i]
        e.name = name.encode()
        e.dev_ptr = t.data_ptr() if t.numel() else 0
        e.nbytes = t.numel() * t.element_size()
        e.ndim = t.dim()
        for d, s in enumerate(t.shape):
            e.shape[d] = s
        e.dtype_code = code
        e.usage = u
        op = post.get(name)
        if op is not None:
            planes = _planes_of(code, u)
            if op[0] == "intdelta":
                e.post_op, e.post_plane = 1, planes - 1
            elif op[0] == "mzs":
                e.post_op, e.post_plane, e.post_k = 2, 0, int(op[1])
            else:
                raise ValueError(f"{name}: unknown per-plane op {op[0]!r}")
        n_planes.append(_planes_of(code, u))
    dev = torch.cuda.current_device() if dev is None else dev
    menu = 0
    for c in cfg.codec_menu:
        if c not in _MENU_BIT:
            raise ValueError(f"codec {c} is not offered by the device encoder (identity, huffman, rans, tans, order1_scale_ac)")
        menu |= _MENU_BIT[c]
    tries = 0
    for c in cfg.candidate_chains:
        if c not in ("intdelta", "mzs"):
            raise ValueError(f"candidate chain {c!r} is not offered by the device encoder (intdelta, mzs)")
        tries |= 1 if c == "intdelta" else 2
    if cfg.shared_states:
        tries |= 4
    opt = _lib.EncodeOptions(_CHUNK_NONE if cfg.streaming_chunk is None else int(cfg.streaming_chunk), menu, -1 if cfg.forced_codec is None else int(cfg.forced_codec), int(cfg.emit_plane_crc),
                             int(cfg.emit_payload_hash), tries)
    torch.cuda.current_stream(dev).synchronize()
    h = C.c_void_p()
    _check(_lib.lib().ptwm_b200_encode_model(arr, len(names), C.byref(opt), dev, stream_handle(dev), C.byref(h)))
    return EncodedContainer(h, names, n_planes, dev)
