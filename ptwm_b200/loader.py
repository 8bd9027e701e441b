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

from . import _lib
from .container import NO_SYNC, ContainerHandle, DecodePlan, PtwmError
from .sharding import contiguous_shards

__all__ = ["PtwmIndex", "plan_shards", "shard_filename", "load_file", "read_sharded_ptwm", "save_sharded", "SafeOpen", "write_mode_b_shell"]

INDEX_NAME = "model.ptwm.index.json"
SINGLE_NAME = "model.ptwm"
_PTWM_SHELL_SIGNAL = "ptwm-shell"
_PTWM_SHELL_TENSOR = "__ptwm_payload__"


# ---- shard bookkeeping ---------------------------------------------------------
_INDEX_FORMAT = "ptwm"
_INDEX_FORMAT_VERSION = 1


@dataclass(frozen=True)
class PtwmIndex:
    """``model.ptwm.index.json``: which shard file holds which tensor.

    The file has the two top-level keys of a safetensors index, so tools that
    collect shard names from ``weight_map`` work on it unchanged; ``metadata``
    adds ``format = "ptwm"``, ``format_version`` and the compressed total beside
    ``total_size`` (behaviour pinned by tests/ptwm/sharding/test_index.py of the
    reference)."""
    total_size: int
    compressed_total_size: int
    weight_map: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return {
            "metadata": {
                "format": _INDEX_FORMAT,
                "format_version": _INDEX_FORMAT_VERSION,
                "total_size": int(self.total_size),
                "compressed_total_size": int(self.compressed_total_size),
            },
            "weight_map": {str(k): str(v) for k, v in self.weight_map.items()},
        }

    @classmethod
    def from_json(cls, doc: Mapping[str, Any], origin="<index>") -> "PtwmIndex":
        header = doc.get("metadata") or {}
        if header.get("format") != _INDEX_FORMAT:
            raise ValueError(f"{origin}: metadata.format={header.get('format')!r}, expected 'ptwm'. This is not a .ptwm index file.")
        return cls(int(header["total_size"]), int(header.get("compressed_total_size", 0)), dict(doc.get("weight_map") or {}))

    def write(self, path) -> None:
        with open(os.fspath(path), "w", encoding="utf-8") as f:
            json.dump(self.to_json(), f, indent=2)

    @classmethod
    def read(cls, path) -> "PtwmIndex":
        with open(os.fspath(path), "r", encoding="utf-8") as f:
            return cls.from_json(json.load(f), origin=path)

    def shard_files(self) -> list[str]:
        """Distinct shard file names, sorted."""
        return sorted(set(self.weight_map.values()))


def shard_filename(idx_one_based: int, total: int, *, suffix: str) -> str:
    """``model-NNNNN-of-MMMMM.<suffix>`` (five digits each, numbering from 1),
    the Hugging Face shard naming."""
    if idx_one_based < 1 or idx_one_based > total:
        raise ValueError(f"shard index {idx_one_based} out of [1, {total}]")
    return "model-%05d-of-%05d.%s" % (idx_one_based, total, suffix)


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
    _idle: list = []          # sets that no load is using, most recently returned last
    _lock = threading.Lock()

    def __init__(self, slot_bytes: int, slots: int):
        self.slot_bytes = slot_bytes
        self.bufs = [torch.empty(slot_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(slots)]
        self.views = [memoryview(b.numpy()) for b in self.bufs]
        self.busy: list = [None] * slots  # event of the last copy that read the slot

    @classmethod
    def checkout(cls, slot_bytes: int, slots: int) -> "_Staging":
        """A set that belongs to the caller alone until ``release``: two loads that
        overlap (two threads, one loader per GPU) never share buffers or slot events."""
        with cls._lock:
            for i, st in enumerate(cls._idle):
                if st.slot_bytes == slot_bytes and len(st.bufs) == slots:
                    return cls._idle.pop(i)
            cls._idle.clear()  # another configuration: let its pinned memory go (nothing is using it)
        return cls(slot_bytes, slots)

    def release(self) -> None:
        for ev in self.busy:
            if ev is not None:
                ev.synchronize()  # no copy still reads these buffers
        self.busy = [None] * len(self.bufs)
        with _Staging._lock:
            _Staging._idle.append(self)
            del _Staging._idle[:-2]  # keep at most two idle sets pinned


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
        self.stage = _Staging.checkout(slot_bytes, slots)
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
        if self.stage is not None:
            self.stage.release()  # waits for the last copies out of the buffers, then hands the set back
            self.stage = None
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
        return PtwmIndex.read(index_path).shard_files()
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
    """``safetensors.safe_open`` look-alike for three kinds of file:

    * a ``.ptwm`` container (by suffix): keys are the container's tensors,
      ``metadata()`` is ``None``;
    * a "ptwm-shell" safetensors file, i.e. one whose metadata says
      ``weights_format = "ptwm-shell"`` and whose only tensor
      ``__ptwm_payload__`` is a whole container: keys are the embedded
      container's tensors, ``metadata()`` is the shell's;
    * any other safetensors file: everything is forwarded to safetensors.

    A container is parsed when the file is opened and nothing is decoded until
    ``get_tensor`` names a tensor; that one tensor is then decoded on the GPU.
    Behaviour pinned by tests/ptwm/integrations/test_mode_a_safe_open.py and
    test_mode_b_shell.py of the reference."""

    def __init__(self, filename, framework: str = "pt", device="cuda") -> None:
        path = os.fspath(filename)
        self._container: Optional[ContainerHandle] = None   # set for .ptwm files and shells
        self._st = None                                      # the safetensors handle, when the file is one
        self._shell_metadata = None
        if path.endswith(".ptwm"):
            self._container = ContainerHandle.from_file(path, device=_device_ordinal(device))
            return
        from safetensors import safe_open
        # opened on the host first: a shell's payload has to be parsed from host memory
        probe = safe_open(path, framework, "cpu")
        info = probe.metadata() or {}
        if info.get("weights_format") == _PTWM_SHELL_SIGNAL:
            self._shell_metadata = info
            self._container = ContainerHandle(probe.get_tensor(_PTWM_SHELL_TENSOR), device=_device_ordinal(device))
            self._st = probe
        else:
            probe.__exit__(None, None, None)
            self._st = safe_open(path, framework, str(device))

    def keys(self) -> list[str]:
        if self._container is not None:
            return self._container.names()
        return list(self._st.keys())

    def metadata(self):
        if self._container is not None:
            return self._shell_metadata  # None for a bare .ptwm file
        return self._st.metadata()

    def get_tensor(self, name: str) -> torch.Tensor:
        if self._container is None:
            return self._st.get_tensor(name)
        if name not in self._container:
            raise KeyError(name)
        return self._container.decode(name)

    def get_slice(self, name: str) -> Any:
        if self._container is not None:
            raise NotImplementedError("get_slice is not supported on .ptwm/ptwm-shell containers")
        return self._st.get_slice(name)

    def __enter__(self) -> "SafeOpen":
        return self

    def __exit__(self, *exc) -> None:
        if self._st is not None:
            self._st.__exit__(*exc)

    def __getattr__(self, name: str) -> Any:
        # only reached for names this class does not define: hand them to safetensors when there is a file of its kind
        st = self.__dict__.get("_st")
        if st is None or self.__dict__.get("_container") is not None:
            raise AttributeError(f"'SafeOpen' has no attribute {name!r} (no underlying safetensors file in .ptwm mode)")
        return getattr(st, name)


def write_mode_b_shell(out_path, ptwm_bytes: bytes) -> None:
    """Wrap a container as a single-tensor ``.safetensors`` file that plain
    safetensors can open: the U8 tensor ``__ptwm_payload__`` holds the container
    bytes, the metadata carries ``weights_format = "ptwm-shell"``,
    ``weights_format_version = "1"`` and ``ptwm_bytes_xxhash64``, the XXH64
    (seed 0) of the container as 16 hex digits."""
    from safetensors.torch import save_file
    data = bytes(ptwm_bytes)
    digest = _lib.xxh64(data)
    body = torch.frombuffer(bytearray(data), dtype=torch.uint8) if data else torch.zeros(0, dtype=torch.uint8)
    save_file({_PTWM_SHELL_TENSOR: body}, os.fspath(out_path),
              metadata={"weights_format": _PTWM_SHELL_SIGNAL, "weights_format_version": "1", "ptwm_bytes_xxhash64": f"{digest:016x}"})
