"""Loading ``.ptwm`` files and sharded model directories straight into GPU memory.

Host-side mirror of the reference's loader-side Python for the decode path:
``read_sharded_ptwm`` (python/ptwm/sharding/_reader.py:13-64), ``PtwmIndex``
(python/ptwm/sharding/_index.py:13-46), ``plan_shards`` / ``shard_filename``
(python/ptwm/sharding/_sharder.py:10-43) and ``SafeOpen``
(python/ptwm/integrations/_safetensors.py:44-135).  Same names, arguments and
error behaviour; what differs is where the tensors land: the reference returns
host bytes decoded by its CPU pool, here a file is streamed
file -> pinned staging buffers -> GPU memory while the pieces that have arrived
are already being decoded by the CUDA kernels, and the results are CUDA
tensors.
"""
from __future__ import annotations

import json
import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable, Mapping, Optional, Sequence

import torch

from .container import NO_SYNC, ContainerHandle, DecodePlan, PtwmError
from .sharding import contiguous_shards

__all__ = ["PtwmIndex", "plan_shards", "shard_filename", "load_file", "read_sharded_ptwm", "save_sharded", "SafeOpen", "write_mode_b_shell"]

INDEX_NAME = "model.ptwm.index.json"
SINGLE_NAME = "model.ptwm"
_PTWM_SHELL_SIGNAL = "ptwm-shell"


# ---- shard bookkeeping ---------------------------------------------------------
@dataclass(frozen=True)
class PtwmIndex:
    """``model.ptwm.index.json``: which shard file holds which tensor."""
    total_size: int
    compressed_total_size: int
    weight_map: dict = field(default_factory=dict)

    def write(self, path) -> None:
        payload = {"metadata": {"total_size": self.total_size, "format": "ptwm", "format_version": 1,
                                "compressed_total_size": self.compressed_total_size},
                   "weight_map": dict(self.weight_map)}
        Path(path).write_text(json.dumps(payload, indent=2))

    @classmethod
    def read(cls, path) -> "PtwmIndex":
        payload = json.loads(Path(path).read_text())
        meta = payload.get("metadata", {})
        fmt = meta.get("format")
        if fmt != "ptwm":
            raise ValueError(f"{path}: metadata.format={fmt!r}, expected 'ptwm'. This is not a .ptwm index file.")
        return cls(total_size=int(meta["total_size"]), compressed_total_size=int(meta.get("compressed_total_size", 0)),
                   weight_map=dict(payload.get("weight_map", {})))


def shard_filename(idx_one_based: int, total: int, *, suffix: str) -> str:
    """``model-NNNNN-of-MMMMM.<suffix>``."""
    if not 1 <= idx_one_based <= total:
        raise ValueError(f"shard index {idx_one_based} out of [1, {total}]")
    return f"model-{idx_one_based:05d}-of-{total:05d}.{suffix}"


def plan_shards(sized_tensors: Sequence[tuple[str, int]], *, max_shard_size: int) -> list[list[tuple[str, int]]]:
    """Tensors in input order, a new shard whenever the next tensor would take
    the running size past ``max_shard_size``; a tensor larger than that gets a
    shard of its own."""
    if max_shard_size <= 0:
        raise ValueError(f"max_shard_size must be positive, got {max_shard_size}")
    shards: list[list[tuple[str, int]]] = [[]]
    size = 0
    for name, nbytes in sized_tensors:
        if shards[-1] and size + nbytes > max_shard_size:
            shards.append([])
            size = 0
        shards[-1].append((name, nbytes))
        size += nbytes
    return [s for s in shards if s]


# ---- pinned staging ---------------------------------------------------------------
class _Staging:
    """A few pinned host buffers that file slices pass through on their way to
    the GPU.  Pinning memory is slow (of the order of a second per few GB), so
    the buffers are small, reused round-robin within a load and kept between
    loads."""
    _cache: dict = {}

    def __init__(self, slot_bytes: int, slots: int):
        self.slot_bytes = slot_bytes
        self.bufs = [torch.empty(slot_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(slots)]
        self.views = [memoryview(b.numpy()) for b in self.bufs]
        self.busy: list = [None] * slots  # event of the last copy that read the slot

    @classmethod
    def get(cls, slot_bytes: int, slots: int) -> "_Staging":
        key = (slot_bytes, slots)
        if key not in cls._cache:
            cls._cache.clear()  # one configuration at a time: pinned memory is not returned to the system quickly
            cls._cache[key] = cls(slot_bytes, slots)
        return cls._cache[key]


def _read_into(fd: int, view: memoryview, offset: int, pool: ThreadPoolExecutor, threads: int) -> None:
    """Fill ``view`` with the file bytes from ``offset`` on, the range cut across the pool's threads (preadv releases the GIL)."""
    n = len(view)
    step = max(1 << 20, -(-n // threads))

    def part(a: int) -> None:
        b = min(a + step, n)
        while a < b:
            got = os.preadv(fd, [view[a:b]], offset + a)
            if got <= 0:
                raise PtwmError("file ended while it was being read (truncated or changed underneath the loader)")
            a += got

    for f in [pool.submit(part, a) for a in range(0, n, step)]:
        f.result()


# ---- one file ----------------------------------------------------------------------
class _FileStream:
    """Bytes [first, last) of a file on their way into one GPU buffer.

    A producer thread reads the range slice by slice into the pinned staging
    buffers (``threads`` reader threads per slice) and enqueues the copy of each
    slice on a copy stream of its own; it publishes how far the copies have
    been enqueued together with the event recorded behind each.  A consumer
    asks ``arrived(hi)`` for the event after which file bytes below ``hi`` are
    in ``blob``."""

    def __init__(self, fd: int, first: int, last: int, dev: torch.device, slot_bytes: int, slots: int, threads: int):
        self.fd, self.first, self.last, self.dev = fd, first, last, dev
        self.slot_bytes, self.slots, self.threads = slot_bytes, slots, threads
        self.blob = torch.empty(max(last - first, 1), dtype=torch.uint8, device=dev)
        self.copier = torch.cuda.Stream(dev)
        self.copier.wait_stream(torch.cuda.current_stream(dev))  # the buffer may be recycled memory that earlier work still reads
        self.stage = _Staging.get(slot_bytes, slots)
        self.progress = threading.Condition()
        self.marks: list = []     # (file offset reached, event recorded after the copy that reached it)
        self.failure: list = []
        self.spent = [0.0, 0.0]   # seconds the producer waited for a free buffer / spent reading the file
        self.seen = 0
        self.thread = threading.Thread(target=self._produce, name="ptwm-b200-file-reader", daemon=True)
        self.thread.start()

    def _produce(self) -> None:
        try:
            torch.cuda.set_device(self.dev)
            stage, sent, k = self.stage, self.first, 0
            with ThreadPoolExecutor(max_workers=self.threads) as pool:
                while sent < self.last:
                    s = k % self.slots
                    k += 1
                    t0 = time.perf_counter()
                    if stage.busy[s] is not None:
                        stage.busy[s].synchronize()  # the copy that last read this buffer has finished
                    t1 = time.perf_counter()
                    n = min(self.slot_bytes, self.last - sent)
                    _read_into(self.fd, stage.views[s][:n], sent, pool, self.threads)
                    self.spent[0] += t1 - t0
                    self.spent[1] += time.perf_counter() - t1
                    with torch.cuda.stream(self.copier):
                        self.blob[sent - self.first:sent - self.first + n].copy_(stage.bufs[s][:n], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(self.copier)
                    stage.busy[s] = ev
                    sent += n
                    with self.progress:
                        self.marks.append((sent, ev))
                        self.progress.notify_all()
        except BaseException as e:  # surfaces in the consuming thread
            with self.progress:
                self.failure.append(e)
                self.progress.notify_all()

    def arrived(self, hi: int):
        """Event after which file bytes [first, hi) are in the blob (None when that range is empty); blocks until the copy is enqueued.
        Calls must come with non-decreasing ``hi``."""
        if hi <= self.first:
            return None
        with self.progress:
            while not self.failure and (not self.marks or self.marks[-1][0] < hi):
                self.progress.wait()
            if self.failure:
                raise self.failure[0]
            while self.marks[self.seen][0] < hi:
                self.seen += 1
            return self.marks[self.seen][1]

    def close(self) -> None:
        self.thread.join()
        self.blob.record_stream(self.copier)
        if self.failure:
            raise self.failure[0]


def _decode_stream(handle: ContainerHandle, stream: _FileStream, indices: Sequence[int], pieces: int) -> list[tuple[str, torch.Tensor]]:
    """Decode the tensors ``indices`` while their bytes are still arriving: the
    tensors are cut into ``pieces`` contiguous runs of records, and a run is
    planned, then decoded on the current stream as soon as the last slice it
    needs has been sent, so reading, the PCIe copy and the decode overlap."""
    infos = handle._infos
    dev = stream.dev
    costs = [infos[i]["compressed"] for i in indices]
    runs = [[indices[j] for j in r] for r in contiguous_shards(costs, max(1, min(pieces, len(indices)))) if len(r)]
    compute = torch.cuda.current_stream(dev)
    flags = handle._flags()
    arena_bytes = [sum((infos[i]["orig_size"] + 255) // 256 * 256 for i in run) for run in runs]
    arena = torch.empty(max(sum(arena_bytes), 1), dtype=torch.uint8, device=dev)
    first = stream.first
    jobs, at = [], 0
    # plans first: their small synchronous copies to the device would otherwise queue behind the file's slices
    plans = [DecodePlan(handle, run) for run in runs]
    for plan in plans:
        plan.prepare(handle.device)
    for plan, nbytes in zip(plans, arena_bytes):
        lo, hi = plan.blob_span
        if plan.out_bytes != nbytes or (hi > lo and (lo < first or hi > stream.last)):
            raise PtwmError("internal: plan layout differs from the tensor infos")
        out = arena[at:at + nbytes]
        at += nbytes
        scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device=dev) if plan.scratch_bytes else None
        event = stream.arrived(hi) if hi > lo else None
        if event is not None:
            compute.wait_event(event)
        plan.run(stream.blob[lo - first:hi - first] if hi > lo else stream.blob[:0], out, scratch, blob_first=lo, flags=flags | NO_SYNC)
        jobs.append((plan, out, scratch))
    result = []
    for plan, out, scratch in jobs:
        plan.finish(handle.device, flags)
        result.extend((infos[i]["name"], v) for i, v in zip(plan.indices, plan.views(out)))
    return result


def load_file(path, device: Optional[int] = None, *, names: Optional[Iterable[str]] = None, pieces: int = 8, verify: bool = True,
              skip_missing: bool = False, slot_bytes: int = 128 << 20, slots: int = 4, threads: int = 16,
              timings: Optional[dict] = None) -> dict[str, torch.Tensor]:
    """Decode a ``.ptwm`` file (either layout) into ``{name: CUDA tensor}``.

    The file is parsed in place through a read-only mapping while its bytes
    already stream file -> pinned staging -> GPU; the pieces that have arrived
    are decoded while the rest is still being read.  ``names`` restricts the
    load to some tensors: the file is then parsed first and only the byte span
    those tensors cover is read.  Tensors whose record carries shape metadata
    come back typed and shaped, the others as uint8 vectors of their raw bytes."""
    t0 = time.perf_counter()
    ordinal = torch.cuda.current_device() if device is None else int(device)
    dev = torch.device("cuda", ordinal)
    fd = os.open(os.fspath(path), os.O_RDONLY)
    stream = None
    try:
        size = os.fstat(fd).st_size
        if names is None and size > 0:  # a whole load needs (nearly) every byte: start reading before the parse
            stream = _FileStream(fd, 0, size, dev, int(slot_bytes), int(slots), int(threads))
        handle = ContainerHandle.from_file(path, skip_missing=skip_missing, device=ordinal, verify=verify)
        t1 = time.perf_counter()
        infos = handle._infos
        indices = sorted(range(len(handle)) if names is None else {handle._idx(n) for n in names})
        if stream is None:
            first = min((infos[i]["first_byte"] for i in indices), default=0)
            last = max((infos[i]["end_byte"] for i in indices), default=0)
            stream = _FileStream(fd, first, max(first, last), dev, int(slot_bytes), int(slots), int(threads))
        pairs = _decode_stream(handle, stream, indices, pieces) if indices else []
    finally:
        try:
            if stream is not None:
                stream.close()
        finally:
            os.close(fd)
    if timings is not None:
        timings.update(parse_ms=(t1 - t0) * 1e3, total_ms=(time.perf_counter() - t0) * 1e3, file_bytes=stream.last - stream.first, slices=len(stream.marks),
                       pieces=min(pieces, max(len(indices), 1)), buffer_wait_ms=stream.spent[0] * 1e3, read_ms=stream.spent[1] * 1e3)
    return dict(pairs)


# ---- a model directory -----------------------------------------------------------
def _shard_names(root: Path) -> list[str]:
    index_path = root / INDEX_NAME
    if index_path.exists():
        return sorted(set(PtwmIndex.read(index_path).weight_map.values()))
    if not (root / SINGLE_NAME).exists():
        raise FileNotFoundError(f"{root}: no {SINGLE_NAME} or {INDEX_NAME}")
    return [SINGLE_NAME]


def read_sharded_ptwm(model_dir, device: Optional[int] = None, *, pieces: int = 8, verify: bool = True, **stream_options) -> dict[str, torch.Tensor]:
    """Every shard listed in ``model.ptwm.index.json`` (or the single
    ``model.ptwm``), decoded into one ``{name: CUDA tensor}`` map.

    Raises FileNotFoundError when the directory holds neither file and
    ValueError when a tensor name appears in more than one shard."""
    root = Path(model_dir)
    state: dict[str, torch.Tensor] = {}
    for shard in _shard_names(root):
        for name, tensor in load_file(root / shard, device, pieces=pieces, verify=verify, **stream_options).items():
            if name in state:
                raise ValueError(f"tensor {name!r} appears in multiple shards; shards must partition the tensor name space")
            state[name] = tensor
    return state


def save_sharded(tensors: Mapping[str, torch.Tensor], out_dir, *, max_shard_size: int = 5 << 30, config=None,
                 usage: Optional[Mapping[str, str]] = None) -> PtwmIndex:
    """Encode CUDA tensors on the GPU into ``model-NNNNN-of-MMMMM.ptwm`` shards
    of at most ``max_shard_size`` raw bytes plus ``model.ptwm.index.json``; a
    model that fits one shard becomes a single ``model.ptwm``."""
    from .compressor import compress_model
    root = Path(out_dir)
    root.mkdir(parents=True, exist_ok=True)
    sized = [(n, t.numel() * t.element_size()) for n, t in tensors.items()]
    shards = plan_shards(sized, max_shard_size=max_shard_size) if sized else []
    weight_map: dict[str, str] = {}
    compressed = 0
    for k, shard in enumerate(shards, start=1):
        fname = SINGLE_NAME if len(shards) == 1 else shard_filename(k, len(shards), suffix="ptwm")
        enc = compress_model({n: tensors[n] for n, _ in shard}, config, usage={n: u for n, u in (usage or {}).items() if n in dict(shard)})
        (root / fname).write_bytes(enc.to_bytes())
        compressed += enc.size
        for n, _ in shard:
            weight_map[n] = fname
    index = PtwmIndex(total_size=sum(s for _, s in sized), compressed_total_size=compressed, weight_map=weight_map)
    if len(shards) != 1:
        index.write(root / INDEX_NAME)
    return index


# ---- safetensors-shaped access ---------------------------------------------------
def _device_ordinal(device) -> Optional[int]:
    if device is None or isinstance(device, int):
        return device
    d = torch.device(device)
    if d.type != "cuda":
        raise ValueError(f"ptwm_b200 decodes on CUDA devices only, got device={device!r}")
    return torch.cuda.current_device() if d.index is None else d.index


class SafeOpen:
    """``safetensors.safe_open`` look-alike that also understands ``.ptwm``
    files (mode A) and ``ptwm-shell`` safetensors files, whose single
    ``__ptwm_payload__`` tensor is a whole container (mode B).  Decoding is
    lazy: the container is parsed on open, a tensor is decoded on the GPU when
    ``get_tensor`` asks for it.  Any other safetensors file is passed through
    to the safetensors library."""

    def __init__(self, filename, framework: str = "pt", device="cuda") -> None:
        self._filename = os.fspath(filename)
        self._framework = framework
        self._device = device
        self._mode_a = Path(self._filename).suffix == ".ptwm"
        self._mode_b = False
        self._ptwm: Optional[ContainerHandle] = None
        self._underlying = None
        if self._mode_a:
            self._ptwm = ContainerHandle.from_file(self._filename, device=_device_ordinal(device))
            return
        from safetensors import safe_open
        self._underlying = safe_open(self._filename, framework, "cpu" if self._is_ptwm_shell_probe() else str(device))
        meta = self._underlying.metadata() or {}
        if meta.get("weights_format") == _PTWM_SHELL_SIGNAL:
            self._mode_b = True
            payload = self._underlying.get_tensor("__ptwm_payload__")
            self._ptwm = ContainerHandle(payload, device=_device_ordinal(device))

    def _is_ptwm_shell_probe(self) -> bool:
        # the shell's payload must land in host memory (the parser reads it there), so peek at the metadata first
        from safetensors import safe_open
        with safe_open(self._filename, self._framework, "cpu") as f:
            return (f.metadata() or {}).get("weights_format") == _PTWM_SHELL_SIGNAL

    def keys(self) -> list[str]:
        return self._ptwm.names() if self._ptwm is not None else list(self._underlying.keys())

    def metadata(self):
        return None if self._mode_a else self._underlying.metadata()

    def get_tensor(self, name: str) -> torch.Tensor:
        if self._ptwm is None:
            return self._underlying.get_tensor(name)
        if name not in self._ptwm:
            raise KeyError(name)
        return self._ptwm.decode(name)

    def get_slice(self, name: str) -> Any:
        if self._ptwm is not None:
            raise NotImplementedError("get_slice is not supported on .ptwm/ptwm-shell containers")
        return self._underlying.get_slice(name)

    def __enter__(self) -> "SafeOpen":
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> None:
        if self._underlying is not None:
            return self._underlying.__exit__(exc_type, exc_value, traceback)
        return None

    def __getattr__(self, name: str) -> Any:
        underlying = self.__dict__.get("_underlying")
        if underlying is None:
            raise AttributeError(f"'SafeOpen' has no attribute {name!r} (no underlying safetensors file in .ptwm mode)")
        return getattr(underlying, name)


def write_mode_b_shell(out_path, ptwm_bytes: bytes) -> None:
    """Wrap a container as a valid single-tensor ``.safetensors`` file: one U8
    tensor ``__ptwm_payload__`` and ``weights_format = "ptwm-shell"`` in the
    metadata."""
    from safetensors.torch import save_file
    payload = torch.frombuffer(bytearray(ptwm_bytes), dtype=torch.uint8).clone()
    save_file({"__ptwm_payload__": payload}, os.fspath(out_path),
              metadata={"weights_format": _PTWM_SHELL_SIGNAL, "weights_format_version": "1"})
