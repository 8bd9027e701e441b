"""Decode throughput of one `.ptwm` container on B200.

Workload: the synthetic Llama-3-8B-shape bf16 state dict (291 tensors,
16.06 GB; weights Normal(0, 0.02), norm vectors 1 + Normal(0, 0.01)), written
as ONE compact container by this package's device encoder the way the
reference's own decode benchmark writes its input (forced rANS, no payload
hash, no plane CRC: benchmarks/decode_throughput.py:41-42 and
benchmarks/_common.py:190-198 of the reference), with 32 KiB chunks.  A step
decodes the whole container; with N ranks the records are split into N
contiguous runs and every rank decodes its own run from its own byte range of
the file, with no collective (strong scaling).

At one GPU the line also carries `extras`: smaller cases of what other writers
produce (plane CRCs and payload hashes verified, 512 KiB chunks, tANS exponent
planes, the full codec menu, the other benchmark configurations with their own
roofline figures, and the encode path), each timed with the L2 flushed between
iterations.  With N ranks it carries `replica_e2e`: every rank ends up with the
whole model (its share of the compressed bytes over PCIe, the rest over NVLink).

  python bench.py --gpus 1 --steps 5 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N
  python bench.py --impl reference      (CPU restatement of the reference decoder)

One JSON line on stdout (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DRAM_BYTES_PER_ALGORITHMIC_BYTE = {"rans_fused": 1.0123, "huffman_fused": 1.0094}

LLAMA8B = dict(layers=32, d=4096, kv=1024, ffn=14336, vocab=128256)


def model_shapes(layers: int, d: int, kv: int, ffn: int, vocab: int):
    """(name, shape, is_norm) in state-dict order."""
    out = [("model.embed_tokens.weight", (vocab, d), False)]
    for i in range(layers):
        p = f"model.layers.{i}."
        out += [(p + "self_attn.q_proj.weight", (d, d), False), (p + "self_attn.k_proj.weight", (kv, d), False),
                (p + "self_attn.v_proj.weight", (kv, d), False), (p + "self_attn.o_proj.weight", (d, d), False),
                (p + "mlp.gate_proj.weight", (ffn, d), False), (p + "mlp.up_proj.weight", (ffn, d), False),
                (p + "mlp.down_proj.weight", (d, ffn), False), (p + "input_layernorm.weight", (d,), True),
                (p + "post_attention_layernorm.weight", (d,), True)]
    out += [("model.norm.weight", (d,), True), ("lm_head.weight", (vocab, d), False)]
    return out


def make_tensor(name_index: int, shape, is_norm: bool, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(1000 + name_index)
    x = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
    x = 1 + 0.01 * x if is_norm else 0.02 * x
    return x.to(torch.bfloat16)


def build_container(shapes, indices, device, chunk: int, codec: str, crc: bool, hash_: bool = False):
    """Encode the tensors `indices` of `shapes` on the device; returns (EncodedContainer, raw bytes)."""
    import ptwm_b200
    from ptwm_b200.compressor import HUFFMAN, IDENTITY, RANS, TANS, CompressionConfig, compress_model
    tensors = {}
    raw = 0
    for i in indices:
        name, shape, is_norm = shapes[i]
        tensors[name] = make_tensor(i, shape, is_norm, device)
        raw += tensors[name].numel() * 2
    forced = {"rans": RANS, "huffman": HUFFMAN, "tans": TANS, "identity": IDENTITY, "auto": None}[codec]
    cfg = CompressionConfig(streaming_chunk=chunk, forced_codec=forced, codec_menu=(IDENTITY, HUFFMAN, RANS), emit_plane_crc=crc, emit_payload_hash=hash_)
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    enc = compress_model(tensors, cfg, device=device.index)
    torch.cuda.synchronize(device)
    enc.encode_s = time.perf_counter() - t0  # the call returns with the container complete in device memory
    return enc, raw, tensors


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def peak_hbm_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def cpu_sample(shapes, device, args, layers: int):
    """Container of the first `layers` transformer layers of the same state dict, as host bytes, plus the expected raw bytes."""
    per_layer = 9
    indices = list(range(1, 1 + per_layer * layers))
    enc, raw, tensors = build_container(shapes, indices, device, args.chunk, args.codec, args.crc, args.hash)
    blob = enc.to_bytes()
    expect = b"".join(t.view(torch.uint8).cpu().numpy().tobytes() for t in tensors.values())
    del enc, tensors
    torch.cuda.empty_cache()
    return blob, raw, expect, f"first {layers} of {LLAMA8B['layers']} transformer layers ({len(indices)} tensors, {raw / 1e9:.2f} GB raw) of the same container recipe"


def time_cpu_decode(blob, expect, threads: int, repeats: int):
    """Seconds per decode_model of the CPU restatement (tensors and chunks across `threads` host threads)."""
    import oracle
    c = oracle.Container(blob)
    n = len(c.tensors)
    dec, sec, data = c.decode_range(0, n, threads=threads, verify=True, keep=True)
    assert data == expect, "CPU restatement decoded different bytes"
    times = []
    for _ in range(repeats):
        dec, sec = c.decode_range(0, n, threads=threads, verify=True, keep=False)
        times.append(sec)
    return statistics.median(times), dec


_FLUSH = {}


def flush_l2(device):
    """Overwrite a buffer larger than the 126 MB L2 so that the next iteration starts with a cold cache."""
    buf = _FLUSH.get(device)
    if buf is None:
        buf = _FLUSH[device] = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    buf.fill_(1)


def sigma_row_weights(rows, cols, seed, device):
    """Normal(0, sigma_row), sigma_row log-uniform in [0.005, 0.05] per row (the block-set configurations)."""
    import math
    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn(rows, cols, generator=g, device=device)
    lo, hi = math.log(0.005), math.log(0.05)
    return w * torch.exp(torch.rand(rows, 1, generator=g, device=device) * (hi - lo) + lo)


def _e2m1_pack(x):
    levels = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=x.device)
    idx = (x.abs().unsqueeze(-1) - levels).abs().argmin(-1).to(torch.uint8) | ((x < 0).to(torch.uint8) << 3)
    return (idx[..., 0::2] | (idx[..., 1::2] << 4)).contiguous()


def config_tensors(which: str, device):
    """Synthetic tensors of the reference's benchmark configurations 1-4 -> (tensors, usage)."""
    d, ffn = 4096, 14336
    if which == "config1":
        return {"w": make_tensor(0, (d, d), False, device)}, {}
    if which in ("config2_fp32", "config2_fp16"):
        dt = torch.float32 if which.endswith("fp32") else torch.float16
        shapes = [("q", d, d), ("k", d, d), ("v", d, d), ("o", d, d), ("gate", ffn, d), ("up", ffn, d), ("down", d, ffn)]
        t = {f"blk.{n}_proj.weight": sigma_row_weights(r, c, 1000 + i, device).to(dt) for i, (n, r, c) in enumerate(shapes)}
        for i, n in enumerate(("input_layernorm", "post_attention_layernorm")):
            g = torch.Generator(device=device).manual_seed(1100 + i)
            t[f"blk.{n}.weight"] = (1 + 0.01 * torch.randn(d, generator=g, device=device)).to(dt)
        return t, {}
    if which == "config3":
        t = {}
        for i, (rows, cols) in enumerate([(ffn, d), (d, ffn)]):
            w = sigma_row_weights(rows, cols, 2000 + i, device)
            scale = w.abs().amax(dim=1, keepdim=True) / 448.0
            t[f"l{i}.weight"] = (w / scale).to(torch.float8_e4m3fn)
            t[f"l{i}.weight_scale"] = scale.reshape(-1).float()
        return t, {}
    if which == "config4":
        rows, cols = ffn, d
        w = sigma_row_weights(rows, cols, 3000, device).double()
        blk = w.reshape(rows, cols // 32, 32)
        e = (127 + torch.ceil(torch.log2(blk.abs().amax(-1).clamp_min(1e-30) / 6.0))).clamp(0, 254).to(torch.uint8)
        mx = _e2m1_pack((blk / torch.exp2(e.double() - 127).unsqueeze(-1)).reshape(rows, cols).float())
        g = w.abs().max() / (448.0 * 6.0)
        blk = w.reshape(rows, cols // 16, 16)
        s8 = (blk.abs().amax(-1) / 6.0 / g).float().to(torch.float8_e4m3fn)
        sc = s8.float().double() * g
        sc = torch.where(sc == 0, torch.ones_like(sc), sc).unsqueeze(-1)
        nv = _e2m1_pack((blk / sc).reshape(rows, cols).float())
        t = {"mx.blocks": mx, "mx.scales": e.contiguous(), "nv.weight": nv, "nv.weight_scale": s8.contiguous(), "nv.weight_scale_2": g.float().reshape(1)}
        return t, {"mx.blocks": "fp4", "mx.scales": "scale", "nv.weight": "fp4", "nv.weight_scale": "scale", "nv.weight_scale_2": "global_scale"}
    raise ValueError(which)


_SLOT_NAMES_DECODE = ("rans", "huffman", "tans", "o1sac", "rans_fused", "huffman_fused", "tans_final", "o1sac_final")


def measure_case(tensors, usage, cfg, device, peak, verify=False, reps=5, check=True):
    """Encode `tensors` on the device, then decode the container from device memory `reps` times with the L2 flushed
    before each, CUDA events around each pass; per-kernel times from separate passes.  Returns one extras entry."""
    import ptwm_b200
    from ptwm_b200.compressor import compress_model
    local = device.index
    raw = sum(t.numel() * t.element_size() for t in tensors.values())
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    enc = compress_model(tensors, cfg, usage=usage, device=local)
    torch.cuda.synchronize()
    encode_s = time.perf_counter() - t0
    blob_dev = enc.to_tensor()
    host = blob_dev.cpu()
    codecs = enc.plane_codecs
    size = enc.size
    del enc
    h = ptwm_b200.ContainerHandle(host, device=local, verify=verify)
    plan = h.plan()
    lo, hi = plan.blob_span
    out = torch.empty(plan.out_bytes, dtype=torch.uint8, device=device)
    scratch = torch.empty(max(plan.scratch_bytes, 1), dtype=torch.uint8, device=device)
    flags = (ptwm_b200.VERIFY_CRC | ptwm_b200.VERIFY_HASH) if verify else 0
    span = blob_dev[lo:hi]
    plan.run(span, out, scratch, blob_first=lo, flags=flags)
    if check:
        for (name, t), v in zip(tensors.items(), plan.views(out)):
            if not torch.equal(v.contiguous().view(torch.uint8).reshape(-1), t.contiguous().view(torch.uint8).reshape(-1)):
                raise SystemExit(f"extras: decoded tensor {name} differs from the source")
    times = []
    for _ in range(2 + reps):
        flush_l2(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        plan.run(span, out, scratch, blob_first=lo, flags=flags | ptwm_b200.NO_SYNC)
        b.record()
        plan.finish(local, flags)
        times.append(a.elapsed_time(b))
    ms = statistics.median(times[2:])
    slot = {}
    for _ in range(3):
        flush_l2(device)
        plan.run(span, out, scratch, blob_first=lo, flags=flags | ptwm_b200.TIME_KERNELS)
        for name, (t, nbytes, items) in plan.timings(local).items():
            slot.setdefault(name, ([], nbytes, items))[0].append(t)
    kernels = {n: {"ms": round(statistics.median(v[0]), 4), "bytes": v[1], "items": v[2]} for n, v in slot.items()}
    entry = {"raw_bytes": int(raw), "compressed_bytes": int(size), "ratio": round(size / max(raw, 1), 4), "ms": round(ms, 4), "value": raw / (ms * 1e-3) / 1e9,
             "unit": "GB/s", "hbm_roofline_frac_whole_pass": (plan.bytes_read + raw) / (ms * 1e-3) / 1e9 / peak, "kernels": kernels,
             "codecs": sorted({str(v) for v in codecs.values()}), "launches": plan.launches}
    dec = {n: k for n, k in kernels.items() if n in _SLOT_NAMES_DECODE or n in ("merge", "crc32", "xxh64")}
    if dec:
        top = max(dec, key=lambda n: dec[n]["ms"])
        ach = dec[top]["bytes"] / (dec[top]["ms"] * 1e-3) / 1e9 if dec[top]["ms"] > 0 else 0.0
        entry["roofline"] = {"bound": "hbm", "kernel": top, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                             "algorithmic_bytes": dec[top]["bytes"], "ms": dec[top]["ms"]}
    entry["encode"] = {"ms": round(encode_s * 1e3, 3), "value": raw / encode_s / 1e9, "unit": "GB/s",
                       "roofline": {"bound": "hbm", "achieved": (raw + size) / encode_s / 1e9, "peak": peak, "unit": "GB/s", "frac": (raw + size) / encode_s / 1e9 / peak,
                                    "what": "raw bytes read + container bytes written over the wall time of compress_model (split, histograms, tables, streams, CRC/hash when asked, gather)"}}
    return entry


def run_extras(shapes, device, args, peak):
    """Bounded samples of what other writers produce and of the other configurations (one GPU only)."""
    from ptwm_b200.compressor import HUFFMAN, IDENTITY, ORDER1_SCALE_AC, RANS, TANS, CompressionConfig
    full = (IDENTITY, HUFFMAN, RANS, TANS, ORDER1_SCALE_AC)
    layers = min(args.cpu_layers, LLAMA8B["layers"])
    sample = {shapes[i][0]: make_tensor(i, shapes[i][1], shapes[i][2], device) for i in range(1, 1 + 9 * layers)}
    what = f"first {layers} transformer layers of the headline state dict"
    out = {}
    cases = {
        "verify": (dict(streaming_chunk=args.chunk, forced_codec=RANS, emit_plane_crc=True, emit_payload_hash=True), True, what + ", written with plane CRC-32s and XXH64 payload hashes, both checked on decode"),
        "chunk_512k": (dict(streaming_chunk=512 << 10, forced_codec=RANS), False, what + ", 512 KiB chunks (the reference benchmark's own chunk size, benchmarks/decode_throughput.py:41-42)"),
        "huffman": (dict(streaming_chunk=args.chunk, forced_codec=HUFFMAN), False, what + ", Huffman exponent planes"),
        "tans_menu": (dict(streaming_chunk=args.chunk, forced_codec=TANS), False, what + ", tANS exponent planes (what the reference's trial encode picks for them)"),
        "full_menu_64k": (dict(streaming_chunk=65536, codec_menu=full, emit_plane_crc=True), True, what + ", codec per plane from the full menu, 64 KiB chunks, plane CRCs checked"),
    }
    for name, (kw, verify, desc) in cases.items():
        e = measure_case(sample, {}, CompressionConfig(**kw), device, peak, verify=verify)
        e["sample"] = desc
        out[name] = e
    del sample
    torch.cuda.empty_cache()
    for which in ("config1", "config2_fp32", "config2_fp16", "config3", "config4"):
        tensors, usage = config_tensors(which, device)
        e = measure_case(tensors, usage, CompressionConfig(streaming_chunk=args.chunk, codec_menu=full), device, peak)
        e["sample"] = f"{which}: shapes and value distributions of the reference's benchmark configuration, full codec menu, {args.chunk // 1024} KiB chunks"
        out[which] = e
        del tensors
        torch.cuda.empty_cache()
    # the scale planes of a large MXFP4 model: enough Order1ScaleAC chunks to fill every SM several times over
    scales, usage = {}, {}
    for i in range(170):
        blk = sigma_row_weights(14336, 4096, 5000 + i, device).reshape(14336, 128, 32)
        scales[f"l{i}.scales"] = (127 + torch.ceil(torch.log2(blk.abs().amax(-1).clamp_min(1e-30) / 6.0))).clamp(0, 254).to(torch.uint8).contiguous()
        usage[f"l{i}.scales"] = "scale"
        del blk
    e = measure_case(scales, usage, CompressionConfig(streaming_chunk=args.chunk, codec_menu=full), device, peak, reps=3)
    e["sample"] = "mx_scales: the E8M0 scale planes of 170 MXFP4 [14336, 4096] projections (312 MB, 9520 chunks), full codec menu: Order1ScaleAC at full occupancy"
    out["mx_scales"] = e
    del scales
    torch.cuda.empty_cache()
    out["l2"] = "a 256 MB buffer is overwritten before every timed pass (config1 and the scale planes are smaller than the 126 MB L2)"
    return out


def reference_wheel():
    """The reference's own package, when one was installed under baseline/_ref (it cannot be built in this image: no Rust toolchain)."""
    path = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(path):
        return None
    sys.path.insert(0, path)
    try:
        import ptwm  # noqa: F401
        from ptwm import _rust
        return _rust
    except Exception:
        return None
    finally:
        sys.path.remove(path)


def run_reference(args):
    """The reference arm: the CPU restatement of ptwm-core's decode_model on the host cores (the Rust crate itself cannot be built in this image)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    shapes = model_shapes(**LLAMA8B)
    threads = oracle.num_procs()
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        blob, raw, expect, sample = cpu_sample(shapes, device, args, args.cpu_layers)
    else:  # no device to run the product encoder on: the oracle's own writer makes a smaller sample
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from _data import spec_bf16
        specs = [spec_bf16(f"w{i}", 1024, 4096, i) for i in range(4)]
        blob = oracle.write_container(specs, chunk_size=args.chunk, forced_codec=oracle.RANS)
        expect = b"".join(s.raw for s in specs)
        raw = len(expect)
        sample = "4 bf16 [1024,4096] tensors written by the oracle (no CUDA device for the product encoder)"
    rust = reference_wheel()
    kind = "port"
    if rust is not None:  # the reference's own decoder, on the same bytes; its output also pins the port (and the device writer) against it
        os.environ.setdefault("RAYON_NUM_THREADS", str(threads))
        decoded = rust.decode_model(blob)
        got = b"".join(bytes(v) for _, v in (decoded.items() if hasattr(decoded, "items") else decoded))
        if got != expect:
            raise SystemExit("the reference decoder and the source tensors disagree on the device-written container")
        run = lambda: rust.decode_model(blob)  # noqa: E731
        kind = "reference"
        sample += f"; ptwm._rust.decode_model, RAYON_NUM_THREADS={os.environ['RAYON_NUM_THREADS']}"
    else:
        c = oracle.Container(blob)
        n = len(c.tensors)
        run = lambda: c.decode_range(0, n, threads=threads, verify=True)  # noqa: E731
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    value = raw / dt / 1e9
    line = {"impl": "reference", "metric": "decoded_GB_per_s", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": workload_config(args, raw_bytes=raw, compressed=len(blob)),
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit_json(line)


def workload_config(args, raw_bytes, compressed):
    return {"workload": "llama3-8b-shape bf16 state dict, one PTWC container" if not args.layers else f"llama3-8b-shape bf16, {args.layers} layers",
            "raw_bytes": raw_bytes, "compressed_bytes": compressed, "ratio": round(compressed / max(raw_bytes, 1), 4), "chunk_bytes": args.chunk, "codec": args.codec,
            "plane_crc": bool(args.crc), "payload_hash": bool(args.hash), "l2": "inputs and outputs far larger than the 126 MB L2 (no flush needed)",
            "parallelism": f"records split over {args.gpus} rank(s), no collective"}


def run_ours(args):
    import torch.distributed as dist
    import ptwm_b200
    from ptwm_b200.sharding import shard_for_rank
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: ptwm_b200 has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = dict(LLAMA8B)
    if args.layers:
        cfg["layers"] = args.layers
    shapes = model_shapes(**cfg)
    if not args.pieces:
        args.pieces = 8
    if args.workload == "c1x16":  # profiling-sized stand-in: sixteen bf16 [4096,4096] tensors (0.54 GB), same recipe
        shapes = [(f"w{i}.weight", (4096, 4096), False) for i in range(16)]
        cfg["layers"] = 0

    # ---- set-up (untimed): synthesize, encode on the device, keep this rank's byte range ----
    t_setup = time.perf_counter()
    enc, raw_total, tensors = build_container(shapes, range(len(shapes)), device, args.chunk, args.codec, args.crc, args.hash)
    compressed = enc.size
    codecs = enc.plane_codecs
    encode_s = enc.encode_s
    host_blob = torch.empty(compressed, dtype=torch.uint8, pin_memory=True)
    blob_dev = enc.to_tensor()
    host_blob.copy_(blob_dev)
    del enc
    handle = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc or args.hash))
    infos = handle.tensor_infos()
    mine = shard_for_rank(infos, rank, world)
    plan = handle.plan(mine)
    lo, hi = plan.blob_span
    span_dev = blob_dev[lo:hi].clone()
    del blob_dev
    out = torch.empty(plan.out_bytes, dtype=torch.uint8, device=device)
    scratch = torch.empty(max(plan.scratch_bytes, 1), dtype=torch.uint8, device=device)
    flags = (ptwm_b200.VERIFY_CRC if args.crc else 0) | (ptwm_b200.VERIFY_HASH if args.hash else 0)

    # parity of this rank's tensors with the source tensors, once, before anything is timed
    plan.run(span_dev, out, scratch, blob_first=lo, flags=flags)
    for i, view in zip(mine, plan.views(out)):
        if not args.no_check and not torch.equal(view.view(torch.uint8), tensors[infos[i]["name"]].view(torch.uint8)):
            raise SystemExit(f"rank {rank}: decoded tensor {infos[i]['name']} differs from the source")
    my_raw = sum(infos[i]["orig_size"] for i in mine)
    del tensors
    torch.cuda.empty_cache()
    setup_s = time.perf_counter() - t_setup

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ---------------------------------------------------------
    for _ in range(args.warmup):
        plan.run(span_dev, out, scratch, blob_first=lo, flags=flags | ptwm_b200.NO_SYNC)
    plan.finish(local, flags)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        plan.run(span_dev, out, scratch, blob_first=lo, flags=flags | ptwm_b200.NO_SYNC)
    end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    plan.finish(local, flags)
    ms = torch.tensor([start.elapsed_time(end)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps

    # ---- per-kernel durations (separate runs, CUDA events around each launch on the same stream) ----
    slot_ms, slot_meta = {}, {}
    reps = 5
    for _ in range(reps):
        plan.run(span_dev, out, scratch, blob_first=lo, flags=flags | ptwm_b200.TIME_KERNELS)
        for name, (t, nbytes, items) in plan.timings(local).items():
            slot_ms.setdefault(name, []).append(t)
            slot_meta[name] = (nbytes, items)
    kernels = {name: {"ms": statistics.mean(v), "bytes": slot_meta[name][0], "items": slot_meta[name][1]} for name, v in slot_ms.items()}
    status_bytes = 4 * (1 + sum(k["items"] for n, k in kernels.items() if n not in ("merge", "copy_to_scratch", "crc32", "xxh64")))

    # ---- end to end: pinned host container -> parse, plan, H2D of the rank's span, decode, status read-back ----
    e2e_times, e2e_parts = [], []
    for it in range(args.warmup + args.steps):
        barrier()
        t0 = time.perf_counter()
        if world == 1:  # one rank needs every byte: start the copy before the parse
            h2 = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc or args.hash), prefetch=True)
            share = mine
        else:  # a rank reads only the records of its shard (a contiguous run cut by record bytes; the shards partition the container)
            h2 = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc or args.hash), shard=(rank, world))
            share = h2.shard_indices()
        t1 = time.perf_counter()
        decoded = h2.decode_model_streamed(indices=share, pieces=args.pieces)
        e2e_tensors = len(decoded)
        t2 = time.perf_counter()
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        if it >= args.warmup:
            e2e_times.append(float(dt.item()))
            e2e_parts.append((t1 - t0, t2 - t1))
        del decoded, h2
    e2e_s = statistics.mean(e2e_times)

    # ---- replica mode (N > 1): every rank ends up with the whole model ------------------------------------------
    replica = None
    if world > 1:
        from ptwm_b200.sharding import decode_replica
        hr = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc or args.hash))
        rep_times, nvlink = [], 0
        for it in range(2 + min(args.steps, 5)):
            barrier()
            t0 = time.perf_counter()
            decoded, nvlink = decode_replica(hr, None)
            torch.cuda.synchronize()
            dt = torch.tensor([time.perf_counter() - t0], device=device, dtype=torch.float64)
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            if it >= 2:
                rep_times.append(float(dt.item()))
            n_rep = len(decoded)
            if it == 0 and not args.no_check:
                # every tensor of the replica against its owner's device-resident decode (checked against the source above):
                # 32-bit word sums, the owners' gathered by a sum over ranks
                def word_sum(t):
                    b = t.contiguous().view(torch.uint8).reshape(-1)
                    n4 = b.numel() // 4 * 4
                    return int(b[:n4].view(torch.int32).sum(dtype=torch.int64).item()) + int(b[n4:].sum(dtype=torch.int64).item())
                got = torch.tensor([word_sum(t) for _, t in decoded], device=device, dtype=torch.int64)
                own = torch.zeros(len(infos), device=device, dtype=torch.int64)
                for i, view in zip(mine, plan.views(out)):
                    own[i] = word_sum(view)
                dist.all_reduce(own, op=dist.ReduceOp.SUM)
                if got.numel() != own.numel() or not torch.equal(got, own):
                    raise SystemExit(f"rank {rank}: replica decode differs from the owners' decode")
            del decoded
        sec = statistics.mean(rep_times)
        replica = {"value": raw_total / sec / 1e9, "unit": "GB/s per replica", "ms_per_step": sec * 1e3, "tensors_per_rank": n_rep,
                   "nvlink_bytes_received_per_rank": int(nvlink), "h2d_bytes_per_rank": int(compressed - nvlink),
                   "includes": "per rank: H2D of its span of the compressed container (1 / N of it), the spans exchanged in four slices each (one NCCL broadcast per slice and owner, into place, while later slices are still crossing PCIe), one full local decode; container already parsed"}
        del hr

    # ---- optional: the same container as a file (page cache warm) -> load_file --------------------------------
    file_load = None
    if args.file_dir and world == 1:
        path = os.path.join(args.file_dir, f"ptwm_b200_bench_{os.getpid()}.ptwm")
        try:
            with open(path, "wb") as f:
                f.write(memoryview(host_blob.numpy()))
            times, info = [], {}
            for it in range(args.warmup + args.steps):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                state = ptwm_b200.load_file(path, local, pieces=8, verify=bool(args.crc or args.hash), threads=args.file_threads, timings=info)
                torch.cuda.synchronize()
                if it >= args.warmup:
                    times.append(time.perf_counter() - t0)
                if it == 0 and not args.no_check:
                    probe = infos[len(infos) // 2]["name"]
                    if not torch.equal(state[probe].view(torch.uint8).reshape(-1), plan.views(out)[mine.index(len(infos) // 2)].view(torch.uint8).reshape(-1)):
                        raise SystemExit("load_file: decoded tensor differs from the device-resident decode")
                del state
            sec = statistics.mean(times)
            file_load = {"value": my_raw / sec / 1e9, "unit": "GB/s", "ms": sec * 1e3, "parse_ms": info.get("parse_ms"), "threads": args.file_threads,
                         "file_bytes": int(compressed), "includes": "load_file(path): file -> pinned staging -> GPU in 128 MiB slices, started before the parse of the mapped file; arrived pieces are decoded while the rest is read"}
        finally:
            if os.path.exists(path):
                os.remove(path)

    totals = torch.tensor([float(my_raw), float(hi - lo), float(plan.bytes_read), float(plan.launches), float(e2e_tensors)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    total_raw, total_h2d, total_read, total_launches, total_e2e_tensors = (float(x) for x in totals.tolist())
    if int(total_e2e_tensors) != len(infos):
        raise SystemExit(f"end-to-end leg decoded {int(total_e2e_tensors)} tensors over all ranks, the container holds {len(infos)}")

    if rank == 0:
        peak, peak_kind = peak_hbm_gbs()
        top = max(kernels, key=lambda n: kernels[n]["ms"]) if kernels else None
        roof = None
        if top:
            k = kernels[top]
            achieved = k["bytes"] / (k["ms"] * 1e-3) / 1e9
            # DRAM bytes (read + written) per algorithmic byte from one ncu capture of the kernel on a smaller case of the
            # same recipe (two transformer layers plus embeddings, 3 GB raw), scaled to this launch: traffic grows with the
            # number of chunks, like the algorithmic bytes.  The captures are summarised under profiles/.
            ratio = DRAM_BYTES_PER_ALGORITHMIC_BYTE.get(top)
            traffic = ratio * k["bytes"] if ratio else None
            roof = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": traffic, "algorithmic_bytes": k["bytes"], "ms": k["ms"]}
        line = {"metric": "decoded_GB_per_s", "value": total_raw / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8",
                "data": "synthetic", "config": workload_config(args, int(raw_total), int(compressed)),
                "hbm_roofline_frac_whole_step": (total_read + total_raw) / world / (ms_per_step * 1e-3) / 1e9 / peak,
                "roofline": roof, "kernels_rank0": kernels, "clocks": clocks,
                "e2e": {"value": total_raw / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(total_h2d), "d2h_bytes_per_step": int(status_bytes * world),
                        "ms_per_step": e2e_s * 1e3,
                        "parts_ms": {"parse": 1e3 * statistics.mean(p[0] for p in e2e_parts), "plan_copy_decode": 1e3 * statistics.mean(p[1] for p in e2e_parts)},
                        "pieces": args.pieces, "h2d_GBps_per_rank": total_h2d / world / max(statistics.mean(p[1] for p in e2e_parts), 1e-9) / 1e9,
                        "includes": "ContainerHandle(pinned host bytes).decode_model_streamed: parse, per piece plan + H2D copy + decode + status read-back, the copies overlapping the rest (at one GPU the copy starts before the parse; at more a rank opens the container with shard=(rank, world) and reads only its own records)"},
                "gpu_launches": int(total_launches) * args.steps, "setup_s": round(setup_s, 1),
                "plane_codecs": sorted({str(v) for v in codecs.values()})}
        if world == 1:
            line["encode"] = {"value": raw_total / encode_s / 1e9, "unit": "GB/s", "ms": encode_s * 1e3,
                              "roofline": {"bound": "hbm", "achieved": (raw_total + compressed) / encode_s / 1e9, "peak": peak, "unit": "GB/s",
                                           "frac": (raw_total + compressed) / encode_s / 1e9 / peak},
                              "what": "compress_model of the whole state dict in device memory (set-up of this run, one pass, wall time): raw bytes read + container bytes written"}
        if file_load:
            line["file_load"] = file_load
        if replica:
            line["replica_e2e"] = replica
        if world == 1 and not args.no_extras and args.workload == "llama8b" and not args.layers:
            del span_dev, out, scratch, plan, handle
            torch.cuda.empty_cache()
            line["extras"] = run_extras(shapes, device, args, peak)
        if args.workload != "llama8b":
            line["config"]["workload"] = "16 x bf16 [4096,4096] (profiling case)"
        if world == 1 and not args.no_cpu and args.workload == "llama8b":
            import oracle
            blob, raw, expect, sample = cpu_sample(shapes, device, args, min(args.cpu_layers, cfg["layers"]))
            threads = oracle.num_procs()
            sec, dec = time_cpu_decode(blob, expect, threads, repeats=3)
            line["cpu_baseline"] = {"value": dec / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample}
        emit_json(line)
    if world > 1:
        dist.destroy_process_group()


_JSON_OUT = None


def emit_json(line: dict) -> None:
    """The one JSON line goes to the real stdout; everything else that writes to
    file descriptor 1 (NCCL prints its version banner there) is sent to stderr."""
    _JSON_OUT.write(json.dumps(line) + "\n")
    _JSON_OUT.flush()


def main():
    global _JSON_OUT
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--chunk", type=int, default=32768, help="plane bytes per chunk")
    ap.add_argument("--codec", choices=["rans", "huffman", "tans", "auto", "identity"], default="rans")
    ap.add_argument("--crc", action="store_true", help="write and verify plane CRC-32s")
    ap.add_argument("--hash", action="store_true", help="write and verify XXH64 payload hashes (serial per tensor: the largest tensor bounds the pass)")
    ap.add_argument("--pieces", type=int, default=0, help="runs of tensors the end-to-end path decodes one after the other as their bytes arrive (0 = 8): all but the last run decode while later bytes are still crossing PCIe")
    ap.add_argument("--layers", type=int, default=0, help="fewer transformer layers than 32 (for quick checks; not the benchmark workload)")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU baseline sample")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra cases (other writers' containers, configurations 1-4, encode)")
    ap.add_argument("--file-dir", default="", help="also write the container to a file in this directory and time ptwm_b200.load_file on it (extra key file_load; N=1 only)")
    ap.add_argument("--file-threads", type=int, default=16, help="reader threads of load_file")
    ap.add_argument("--no-check", action="store_true", help="skip the parity check (only for timing experimental kernel builds; never for a reported number)")
    ap.add_argument("--workload", choices=["llama8b", "c1x16"], default="llama8b", help="c1x16: small case for profiler captures, not a benchmark line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
