"""Container handle, decompressor and random-access index on CUDA.

Host-side mirror of the reference's Python surface for the decode path:
``ContainerHandle`` (crates/ptwm-py/src/handle.rs:157-227), ``Decompressor``
(python/ptwm/core/_decompressor.py:38-139) and ``TensorIndex``
(python/ptwm/random_access/__init__.py:36-143).  Same method names and
argument meaning; the difference is where the bytes land: decoded tensors are
CUDA ``torch.Tensor`` objects produced by the kernels in ``libptwm_b200.so``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Iterable, Iterator, Optional, Sequence

import torch

from . import _lib
from ._config import DecompressionConfig, HeaderParseError, InvalidDTypeError

MAGIC_PTWS = b"\x89PTWS"
MAGIC_PTWC = b"\x89PTWC\r\n\x1a\n"
MAGIC_PTWM = b"\x89PTWM\r\n\x1a\n"
MAGIC_PTWX = b"\x89PTWX\r\n\x1a\n"

# public dtype codes (crates/ptwm-core/src/dtype.rs:25-50)
_TORCH_DTYPES = {1: torch.float32, 2: torch.float32, 4: torch.float16, 5: torch.float16, 6: torch.bfloat16, 13: torch.uint8, 15: torch.uint32,
                 17: torch.int8, 18: torch.int16, 19: torch.int16, 20: torch.int32, 21: torch.int32, 22: torch.int64, 23: torch.int64,
                 24: torch.bool, 29: torch.float8_e4m3fn, 30: torch.float8_e5m2}
if hasattr(torch, "float4_e2m1fn_x2"):
    _TORCH_DTYPES[31] = torch.float4_e2m1fn_x2

VERIFY_CRC, VERIFY_HASH, NO_SYNC, TIME_KERNELS = 1, 2, 4, 8
SLOT_NAMES = ("rans", "huffman", "tans", "o1sac", "copy_to_scratch", "rans_fused", "huffman_fused", "tans_final", "o1sac_final", "merge", "crc32", "xxh64")


class PtwmError(RuntimeError):
    """A core decode error (the reference surfaces these as RuntimeError, crates/ptwm-py/src/handle.rs:46-48)."""


def _check(rc: int) -> int:
    if rc < 0:
        msg = _lib.last_error()
        raise PtwmError(msg if msg else f"libptwm_b200 error {rc}")
    return rc


def _as_u8_tensor(data) -> torch.Tensor:
    """Host uint8 view of a bytes-like object or tensor, without copying where possible."""
    if isinstance(data, torch.Tensor):
        t = data.contiguous().view(torch.uint8).reshape(-1)
        return t
    mv = memoryview(data)
    if mv.nbytes == 0:
        return torch.empty(0, dtype=torch.uint8)
    if mv.readonly:
        return torch.frombuffer(bytearray(mv), dtype=torch.uint8)
    return torch.frombuffer(mv, dtype=torch.uint8)


def stream_handle(device: int) -> int:
    """cudaStream_t of torch's current stream as an integer the C ABI takes.
    The legacy default stream has handle 0, which the ABI reserves for "the
    library's own stream", so it is passed as cudaStreamLegacy (1)."""
    s = torch.cuda.current_stream(device).cuda_stream
    return s if s else 1


class DecodePlan:
    """Launch plan for a subset of tensors of one container (ptwm_b200_plan)."""

    def __init__(self, handle: "ContainerHandle", indices: Optional[Sequence[int]] = None):
        self.handle = handle
        L = _lib.lib()
        p = C.c_void_p()
        if indices is None:
            self.indices = list(range(len(handle)))
            _check(L.ptwm_b200_plan_create(handle._h, None, 0, C.byref(p)))
        else:
            self.indices = [int(i) for i in indices]
            arr = (C.c_uint32 * max(len(self.indices), 1))(*self.indices)
            _check(L.ptwm_b200_plan_create(handle._h, arr, len(self.indices), C.byref(p)))
        self._p = p
        self.out_bytes = L.ptwm_b200_plan_out_bytes(p)
        self.scratch_bytes = L.ptwm_b200_plan_scratch_bytes(p)
        self.out_offsets = [L.ptwm_b200_plan_out_offset(p, k) for k in range(len(self.indices))]
        lo, hi = C.c_uint64(), C.c_uint64()
        L.ptwm_b200_plan_blob_span(p, C.byref(lo), C.byref(hi))
        self.blob_span = (lo.value, hi.value)
        r, w, n = C.c_uint64(), C.c_uint64(), C.c_uint32()
        L.ptwm_b200_plan_stats(p, C.byref(r), C.byref(w), C.byref(n))
        self.bytes_read, self.bytes_written, self.launches = r.value, w.value, n.value

    def __del__(self):
        if getattr(self, "_p", None):
            _lib.lib().ptwm_b200_plan_destroy(self._p)
            self._p = None
        self._dev_mem = None  # after the plan: its runs are over

    def run(self, blob_dev: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor], *, blob_first: int = 0, flags: int = 0,
            stream: Optional[int] = None) -> None:
        """Enqueue (and unless NO_SYNC is set, finish) one decode pass.
        ``blob_dev`` holds file bytes [blob_first, blob_first + len)."""
        dev = out.device.index if out.device.index is not None else torch.cuda.current_device()
        if stream is None:
            stream = stream_handle(dev)
        sp = scratch.data_ptr() if scratch is not None and scratch.numel() else 0
        sc = scratch.numel() if scratch is not None else 0
        _check(_lib.lib().ptwm_b200_plan_run(self._p, (blob_dev.data_ptr() - blob_first) if blob_dev.numel() else 0, blob_first, blob_dev.numel(),
                                             out.data_ptr() if out.numel() else 0, out.numel(), sp, sc, flags, dev, stream))

    def prepare(self, device: int) -> None:
        """Send the work lists to the device now rather than in the first run.  Their device memory comes from
        torch's allocator (no cudaMalloc, which may wait for transfers that are already queued) and lives as long as the plan."""
        L = _lib.lib()
        if getattr(self, "_dev_mem", None) is None:
            self._dev_mem = torch.empty(int(L.ptwm_b200_plan_device_bytes(self._p)), dtype=torch.uint8, device=torch.device("cuda", device))
            _check(L.ptwm_b200_plan_prepare_in(self._p, device, self._dev_mem.data_ptr(), self._dev_mem.numel()))
        else:
            _check(L.ptwm_b200_plan_prepare(self._p, device))

    def finish(self, device: int, flags: int = 0, stream: Optional[int] = None) -> None:
        if stream is None:
            stream = stream_handle(device)
        _check(_lib.lib().ptwm_b200_plan_finish(self._p, flags, device, stream))

    def timings(self, device: int) -> dict:
        """{slot name: (milliseconds, algorithmic bytes, items)} of the last run made with TIME_KERNELS."""
        ms, by, it = (C.c_float * 12)(), (C.c_uint64 * 12)(), (C.c_uint32 * 12)()
        _check(_lib.lib().ptwm_b200_plan_timings(self._p, device, ms, by, it))
        return {SLOT_NAMES[s]: (ms[s], by[s], it[s]) for s in range(12) if ms[s] >= 0}

    def views(self, out: torch.Tensor) -> list[torch.Tensor]:
        """Typed, shaped views of the planned tensors inside the output arena."""
        return [self.handle._view(i, out, off) for i, off in zip(self.indices, self.out_offsets)]


class ContainerHandle:
    """An opened container: parsed once on the host, decoded on the GPU.

    ``device`` is the CUDA ordinal; the compressed bytes are copied there on
    first use and stay resident for later random-access decodes.  With
    ``prefetch`` (and a buffer in pinned host memory) the copy of the whole
    container to the GPU is started before the container is parsed, in slices
    on a stream of its own, so that the parse costs no time on the way to
    ``decode_model_streamed``.  ``shard=(rank, world)`` reads only that rank's
    share of the tensor records (a contiguous run cut by record bytes; the
    shards of all ranks partition the container), which is what a rank of a
    multi-GPU load needs and costs a world-th of the parse."""

    def __init__(self, buffer, skip_missing: bool = False, device: Optional[int] = None, verify: bool = True, prefetch: bool = False,
                 shard: Optional[tuple] = None):
        resident = None
        if isinstance(buffer, torch.Tensor) and buffer.is_cuda:  # a container already in device memory: parsed from a host copy, decoded where it lies
            resident = buffer.contiguous().view(torch.uint8).reshape(-1)
            buffer = resident.cpu()
        self._host = _as_u8_tensor(buffer)
        self._prefetch = None
        n = self._host.numel()
        if n < len(MAGIC_PTWS):
            raise HeaderParseError("too short to be a .ptwm container")
        head = bytes(self._host[:9].tolist())
        if not (head.startswith(MAGIC_PTWS) or head.startswith(MAGIC_PTWC) or head.startswith(MAGIC_PTWM) or head.startswith(MAGIC_PTWX)):
            raise HeaderParseError("not a .ptwm container")
        self._layout = "compact" if (head.startswith(MAGIC_PTWS) or head.startswith(MAGIC_PTWC)) else "legacy"
        self.device = torch.cuda.current_device() if device is None else int(device)
        if prefetch and self._host.is_pinned():
            self._start_prefetch()
        self._h = C.c_void_p()
        if shard is None:
            _check(_lib.lib().ptwm_b200_open(self._host.data_ptr(), n, C.byref(self._h)))
        else:  # (rank, world): only this rank's records are read, see shard_indices()
            _check(_lib.lib().ptwm_b200_open_shard(self._host.data_ptr(), n, int(shard[0]), int(shard[1]), C.byref(self._h)))
        self.shard = shard
        self.verify = verify
        self.skip_missing = skip_missing
        self._infos = []
        L = _lib.lib()
        for i in range(L.ptwm_b200_tensor_count(self._h)):
            ti = _lib.TensorInfo()
            _check(L.ptwm_b200_tensor_info_get(self._h, i, C.byref(ti)))
            self._infos.append(dict(name=ti.name.decode(), dtype_name=ti.dtype_name.decode(), dtype_code=ti.dtype_code,
                                    shape=[ti.shape[d] for d in range(ti.ndim)] if ti.has_shape else None, has_hash=bool(ti.has_hash),
                                    has_crc=bool(ti.has_crc), supported=bool(ti.supported), kind=ti.kind, orig_size=ti.orig_size,
                                    compressed=ti.compressed, first_byte=ti.first_byte, end_byte=ti.end_byte,
                                    unsupported_reason=ti.unsupported_reason.decode()))
        if not skip_missing:
            for inf in self._infos:
                if not inf["supported"] and "third-party" in inf["unsupported_reason"]:
                    raise ValueError(f"container references an extension that is not installed: {inf['unsupported_reason']}")
        self._index = {inf["name"]: i for i, inf in enumerate(self._infos)}
        self._blob_dev: Optional[torch.Tensor] = resident if resident is not None and resident.device.index == self.device else None
        self._plans: dict = {}

    @classmethod
    def from_file(cls, path, skip_missing: bool = False, device: Optional[int] = None, verify: bool = True) -> "ContainerHandle":
        """Open a container file through a private read-only mapping: the
        parser reads the page cache in place, nothing is copied until a decode
        sends the bytes it needs to the GPU."""
        import mmap
        with open(path, "rb") as f:
            size = f.seek(0, 2)
            if size == 0:
                raise HeaderParseError("too short to be a .ptwm container")
            # ACCESS_COPY gives the writable buffer torch.frombuffer asks for; no page is ever written
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        self = cls(torch.frombuffer(mm, dtype=torch.uint8), skip_missing, device, verify)
        self._mmap = mm
        self.path = Path(path)
        return self

    def __del__(self):
        self._plans = {}
        if getattr(self, "_h", None):
            _lib.lib().ptwm_b200_close(self._h)
            self._h = None

    # -- inspection (handle.rs:168-227) ---------------------------------------
    @property
    def layout(self) -> str:
        return self._layout

    def names(self) -> list[str]:
        return [inf["name"] for inf in self._infos]

    def __len__(self) -> int:
        return len(self._infos)

    def __contains__(self, name: str) -> bool:
        return name in self._index

    def info(self, name: str):
        """(shape, dtype_name, dtype_code, input_format) or None without shape metadata."""
        inf = self._infos[self._idx(name)]
        if inf["shape"] is None:
            return None
        return (list(inf["shape"]), inf["dtype_name"], inf["dtype_code"], 2)

    def shape(self, name: str):
        inf = self._infos[self._idx(name)]
        return None if inf["shape"] is None else (list(inf["shape"]), inf["dtype_name"])

    def shard_indices(self) -> list[int]:
        """Tensors this handle can decode: all supported ones, which for a handle opened with
        ``shard=(rank, world)`` are the supported tensors of that rank's contiguous run of records."""
        return [i for i, inf in enumerate(self._infos) if inf["supported"]]

    def tensor_infos(self) -> list[dict]:
        return [dict(i) for i in self._infos]

    def _idx(self, name) -> int:
        if isinstance(name, int):
            return name
        try:
            return self._index[name]
        except KeyError:
            raise KeyError(name) from None

    # -- device residency -------------------------------------------------------
    def _start_prefetch(self, slice_bytes: int = 64 << 20) -> None:
        dev = torch.device("cuda", self.device)
        n = self._host.numel()
        blob = torch.empty(n, dtype=torch.uint8, device=dev)
        copier = torch.cuda.Stream(dev)
        copier.wait_stream(torch.cuda.current_stream(dev))  # the buffer may be recycled memory that earlier work still reads
        step = slice_bytes  # small enough that nothing else queued on the copy engine waits long behind one
        marks = []  # (file offset reached, event recorded after the copy that reached it)
        with torch.cuda.stream(copier):
            for a in range(0, n, step):
                b = min(a + step, n)
                blob[a:b].copy_(self._host[a:b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copier)
                marks.append((b, ev))
        self._prefetch = (blob, copier, marks)

    def blob_on_device(self) -> torch.Tensor:
        if self._blob_dev is None:
            if self._prefetch is not None:
                blob, copier, marks = self._prefetch
                torch.cuda.current_stream(blob.device).wait_stream(copier)
                blob.record_stream(torch.cuda.current_stream(blob.device))
                self._blob_dev = blob
            else:
                self._blob_dev = self._host.to(torch.device("cuda", self.device))
        return self._blob_dev

    def plan(self, indices: Optional[Sequence[int]] = None) -> DecodePlan:
        key = None if indices is None else tuple(int(i) for i in indices)
        if key not in self._plans:
            self._plans[key] = DecodePlan(self, indices)
        return self._plans[key]

    def _flags(self) -> int:
        return (VERIFY_CRC | VERIFY_HASH) if self.verify else 0

    def _view(self, i: int, out: torch.Tensor, off: int) -> torch.Tensor:
        inf = self._infos[i]
        raw = out[off:off + inf["orig_size"]]
        if inf["shape"] is None:
            return raw
        dt = _TORCH_DTYPES.get(inf["dtype_code"])
        if dt is None:
            raise InvalidDTypeError(f"dtype_code={inf['dtype_code']} has no torch.dtype mapping")
        try:
            return raw.view(dt).reshape(inf["shape"])
        except (RuntimeError, TypeError):
            # packed sub-byte dtypes some torch builds cannot view or reshape: hand back the bytes in shape
            return raw.reshape(inf["shape"]) if dt.itemsize == 1 else raw

    # -- decode (handle.rs:184-193) --------------------------------------------
    def decode_raw(self, name) -> torch.Tensor:
        """Decoded bytes of one tensor as a CUDA uint8 tensor."""
        i = self._idx(name)
        plan = self.plan([i])
        dev = torch.device("cuda", self.device)
        out = torch.empty(plan.out_bytes, dtype=torch.uint8, device=dev)
        scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device=dev) if plan.scratch_bytes else None
        plan.run(self.blob_on_device(), out, scratch, flags=self._flags())
        return out[:self._infos[i]["orig_size"]]

    def decode(self, name) -> torch.Tensor:
        """One tensor, typed and shaped when the record carries shape metadata."""
        i = self._idx(name)
        raw = self.decode_raw(i)
        return self._view(i, raw, 0)

    def decode_model(self, names: Optional[Iterable[str]] = None) -> list[tuple[str, torch.Tensor]]:
        """Every tensor (or the named ones) in one batched pass; the tensors
        are views into one output arena (ContainerReader::decode_model)."""
        indices = None if names is None else [self._idx(n) for n in names]
        plan = self.plan(indices)
        dev = torch.device("cuda", self.device)
        out = torch.empty(plan.out_bytes, dtype=torch.uint8, device=dev)
        scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device=dev) if plan.scratch_bytes else None
        plan.run(self.blob_on_device(), out, scratch, flags=self._flags())
        return [(self._infos[i]["name"], v) for i, v in zip(plan.indices, plan.views(out))]


    def decode_model_streamed(self, names: Optional[Iterable[str]] = None, pieces: int = 8,
                              indices: Optional[Sequence[int]] = None) -> list[tuple[str, torch.Tensor]]:
        """decode_model for a container that is still in host memory (pinned,
        for the copies to run asynchronously): the tensors are cut into
        ``pieces`` contiguous runs of records; the bytes of run k+1 travel to
        the GPU on a copy stream while run k is planned on the host and decoded
        on the current stream, so only the first plan and the last decode are
        not hidden behind the PCIe copy.  Nothing of the container stays
        resident afterwards, unless the handle was opened with ``prefetch``:
        then the copy is already under way and only waited for here."""
        from .sharding import contiguous_shards
        if indices is None:
            indices = list(range(len(self._infos))) if names is None else [self._idx(n) for n in names]
        indices = sorted(int(i) for i in indices)
        if not indices:
            return []
        dev = torch.device("cuda", self.device)
        costs = [self._infos[i]["compressed"] for i in indices]
        runs = [[indices[j] for j in r] for r in contiguous_shards(costs, max(1, min(pieces, len(indices)))) if len(r)]
        compute = torch.cuda.current_stream(dev)
        flags = self._flags()
        # one buffer for the compressed bytes and one arena for the tensors; the pieces are slices of them
        first = min(self._infos[i]["first_byte"] for i in indices)
        last = max(self._infos[i]["end_byte"] for i in indices)
        prefetched = self._prefetch
        if prefetched is not None:
            blob, copier, marks = prefetched
            first = 0
        else:
            copier = torch.cuda.Stream(dev)
            blob = torch.empty(max(last - first, 1), dtype=torch.uint8, device=dev)
        arena_bytes = [sum((self._infos[i]["orig_size"] + 255) // 256 * 256 for i in run) for run in runs]
        arena = torch.empty(max(sum(arena_bytes), 1), dtype=torch.uint8, device=dev)
        copier.wait_stream(compute)  # the buffers may be recycled memory that earlier work on this stream still reads
        jobs, result, at = [], [], 0
        # every plan is made and sent to the device before the first launch: its small synchronous copies would
        # otherwise queue behind the container's slices on the copy engine and hold back the launches of later pieces
        plans = [DecodePlan(self, run) for run in runs]
        for plan in plans:
            plan.prepare(self.device)
        for plan, nbytes in zip(plans, arena_bytes):
            lo, hi = plan.blob_span
            if plan.out_bytes != nbytes or lo < first or hi > last:
                raise PtwmError("internal: plan layout differs from the tensor infos")
            if prefetched is not None:
                arrived = next(ev for end, ev in marks if end >= hi) if hi > 0 else marks[0][1]
            else:
                with torch.cuda.stream(copier):
                    blob[lo - first:hi - first].copy_(self._host[lo:hi], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(copier)
            out = arena[at:at + nbytes]
            at += nbytes
            scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device=dev) if plan.scratch_bytes else None
            compute.wait_event(arrived)
            plan.run(blob[lo - first:hi - first], out, scratch, blob_first=lo, flags=flags | NO_SYNC)
            jobs.append((plan, out, scratch))
        for plan, out, scratch in jobs:
            plan.finish(self.device, flags)
            result.extend((self._infos[i]["name"], v) for i, v in zip(plan.indices, plan.views(out)))
        blob.record_stream(copier)
        return result


class Decompressor:
    """Stateless decompressor; ``decompress`` returns a CUDA tensor."""

    def __init__(self, config: Optional[DecompressionConfig] = None) -> None:
        self.config = config or DecompressionConfig()

    def decompress(self, data) -> torch.Tensor:
        if self.config.codec is not None:
            raise ValueError(f"DecompressionConfig.codec={self.config.codec!r} is set, but decoding always dispatches on the codec "
                             "recorded in the container; leave codec unset.")
        if self.config.delta_second_data is not None:
            raise ValueError("tensor was not compressed using delta compression, but delta_second_data was provided.")
        mv = memoryview(data) if not isinstance(data, torch.Tensor) else None
        if mv is not None and mv.nbytes < len(MAGIC_PTWS):
            raise HeaderParseError("too short to be a .ptwm container")
        handle = ContainerHandle(data, self.config.skip_missing, device=self.config.device, verify=self.config.verify)
        if "_" not in handle:
            raise PtwmError("container holds no tensor named '_'")
        return handle.decode("_")


class TensorEntry:
    """One entry of a ``.ptwm`` tensor index (``python/ptwm/random_access/__init__.py:29-33``): the name, as in the reference."""

    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        object.__setattr__(self, "name", name)

    def __setattr__(self, key, value):
        raise AttributeError("TensorEntry is read-only")

    def __eq__(self, other) -> bool:
        return isinstance(other, TensorEntry) and other.name == self.name

    def __hash__(self) -> int:
        return hash(("TensorEntry", self.name))

    def __repr__(self) -> str:
        return f"TensorEntry(name={self.name!r})"


class TensorIndex:
    """Name-indexed random-access loader over a ``.ptwm`` container file."""

    def __init__(self, path, device: Optional[int] = None, verify: bool = True) -> None:
        self._path = Path(path)
        with open(self._path, "rb") as f:
            head = f.read(9)
        if not (head.startswith(MAGIC_PTWC) or head.startswith(MAGIC_PTWM) or head.startswith(MAGIC_PTWX)):
            raise ValueError(f"{self._path} is not a .ptwm container")
        self._handle = ContainerHandle.from_file(self._path, device=device, verify=verify)
        self._names = self._handle.names()

    @classmethod
    def open(cls, path, device: Optional[int] = None):
        return cls(path, device=device)

    @property
    def path(self) -> Path:
        return self._path

    @property
    def layout(self) -> str:
        return self._handle.layout

    def names(self) -> list[str]:
        return list(self._names)

    def entries(self) -> list[TensorEntry]:
        """Every entry in write order (``random_access/__init__.py:78-80``)."""
        return [TensorEntry(n) for n in self._names]

    def entry(self, name: str) -> TensorEntry:
        if name not in self._handle:
            raise KeyError(name)
        return TensorEntry(name)

    def get_bytes(self, name: str) -> bytes:
        if name not in self._handle:
            raise KeyError(name)
        return bytes(self._handle.decode_raw(name).cpu().numpy().tobytes())

    def get_tensor(self, name: str) -> torch.Tensor:
        if name not in self._handle:
            raise KeyError(name)
        if self._handle.shape(name) is None:
            raise TypeError(f"tensor {name!r} has no shape metadata; cannot reconstruct a torch.Tensor. Call get_bytes().")
        return self._handle.decode(name)

    def stream_tensors(self, names: Optional[Iterable[str]] = None) -> Iterator[tuple[str, torch.Tensor]]:
        for name in (list(names) if names is not None else self.names()):
            yield name, self.get_tensor(name)

    def __len__(self) -> int:
        return len(self._names)

    def __contains__(self, name: str) -> bool:
        return name in self._handle

    def __iter__(self) -> Iterator[str]:
        return iter(self._names)

    def __repr__(self) -> str:
        return f"TensorIndex(path={self._path!s}, n={len(self)})"
