"""Decode throughput of one `.ptwm` container on B200.

Workload: the synthetic Llama-3-8B-shape bf16 state dict (291 tensors,
16.06 GB; weights Normal(0, 0.02), norm vectors 1 + Normal(0, 0.01)), written
as ONE compact container by this package's device encoder the way the
reference's own decode benchmark writes its input (forced rANS, no payload
hash, no plane CRC: benchmarks/decode_throughput.py:41-42 and
benchmarks/_common.py:190-198 of the reference), with 64 KiB chunks.  A step
decodes the whole container; with N ranks the records are split into N
contiguous runs and every rank decodes its own run from its own byte range of
the file, with no collective (strong scaling).

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


def build_container(shapes, indices, device, chunk: int, codec: str, crc: bool):
    """Encode the tensors `indices` of `shapes` on the device; returns (EncodedContainer, raw bytes)."""
    import ptwm_b200
    from ptwm_b200.compressor import HUFFMAN, IDENTITY, RANS, CompressionConfig, compress_model
    tensors = {}
    raw = 0
    for i in indices:
        name, shape, is_norm = shapes[i]
        tensors[name] = make_tensor(i, shape, is_norm, device)
        raw += tensors[name].numel() * 2
    forced = {"rans": RANS, "huffman": HUFFMAN, "identity": IDENTITY, "auto": None}[codec]
    cfg = CompressionConfig(streaming_chunk=chunk, forced_codec=forced, codec_menu=(IDENTITY, HUFFMAN, RANS), emit_plane_crc=crc, emit_payload_hash=False)
    enc = compress_model(tensors, cfg, device=device.index)
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
    enc, raw, tensors = build_container(shapes, indices, device, args.chunk, args.codec, args.crc)
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
    c = oracle.Container(blob)
    n = len(c.tensors)
    for _ in range(args.warmup):
        c.decode_range(0, n, threads=threads, verify=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        c.decode_range(0, n, threads=threads, verify=True)
    dt = (time.perf_counter() - t0) / args.steps
    value = raw / dt / 1e9
    line = {"impl": "reference", "metric": "decoded_GB_per_s", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": workload_config(args, raw_bytes=raw, compressed=len(blob)),
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit_json(line)


def workload_config(args, raw_bytes, compressed):
    return {"workload": "llama3-8b-shape bf16 state dict, one PTWC container" if not args.layers else f"llama3-8b-shape bf16, {args.layers} layers",
            "raw_bytes": raw_bytes, "compressed_bytes": compressed, "ratio": round(compressed / max(raw_bytes, 1), 4), "chunk_bytes": args.chunk, "codec": args.codec,
            "plane_crc": bool(args.crc), "payload_hash": False, "l2": "inputs and outputs far larger than the 126 MB L2 (no flush needed)",
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
        args.pieces = 1 if world == 1 else 8
    if args.workload == "c1x16":  # profiling-sized stand-in: sixteen bf16 [4096,4096] tensors (0.54 GB), same recipe
        shapes = [(f"w{i}.weight", (4096, 4096), False) for i in range(16)]
        cfg["layers"] = 0

    # ---- set-up (untimed): synthesize, encode on the device, keep this rank's byte range ----
    t_setup = time.perf_counter()
    enc, raw_total, tensors = build_container(shapes, range(len(shapes)), device, args.chunk, args.codec, args.crc)
    compressed = enc.size
    codecs = enc.plane_codecs
    host_blob = torch.empty(compressed, dtype=torch.uint8, pin_memory=True)
    blob_dev = enc.to_tensor()
    host_blob.copy_(blob_dev)
    del enc
    handle = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc))
    infos = handle.tensor_infos()
    mine = shard_for_rank(infos, rank, world)
    plan = handle.plan(mine)
    lo, hi = plan.blob_span
    span_dev = blob_dev[lo:hi].clone()
    del blob_dev
    out = torch.empty(plan.out_bytes, dtype=torch.uint8, device=device)
    scratch = torch.empty(max(plan.scratch_bytes, 1), dtype=torch.uint8, device=device)
    flags = ptwm_b200.VERIFY_CRC if args.crc else 0

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
            h2 = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc), prefetch=True)
            share = mine
        else:  # a rank reads only the records of its shard (a contiguous run cut by record bytes; the shards partition the container)
            h2 = ptwm_b200.ContainerHandle(host_blob, device=local, verify=bool(args.crc), shard=(rank, world))
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
                state = ptwm_b200.load_file(path, local, pieces=8, verify=bool(args.crc), threads=args.file_threads, timings=info)
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
                        "pieces": args.pieces,
                        "includes": "ContainerHandle(pinned host bytes).decode_model_streamed: parse, per piece plan + H2D copy + decode + status read-back, the copies overlapping the rest (at one GPU the copy starts before the parse; at more a rank opens the container with shard=(rank, world) and reads only its own records)"},
                "gpu_launches": int(total_launches) * args.steps, "setup_s": round(setup_s, 1),
                "plane_codecs": sorted({str(v) for v in codecs.values()})}
        if file_load:
            line["file_load"] = file_load
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
    ap.add_argument("--codec", choices=["rans", "huffman", "auto", "identity"], default="rans")
    ap.add_argument("--crc", action="store_true", help="write and verify plane CRC-32s")
    ap.add_argument("--pieces", type=int, default=0, help="runs of tensors the end-to-end path decodes one after the other as their bytes arrive; 0 = 1 at one GPU, where the whole copy is started before the parse and a decode beside it only stretched the copy (213 ms with 1 piece, 219 with 4, 227 with 8), else 8")
    ap.add_argument("--layers", type=int, default=0, help="fewer transformer layers than 32 (for quick checks; not the benchmark workload)")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU baseline sample")
    ap.add_argument("--no-cpu", action="store_true")
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
