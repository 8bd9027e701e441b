"""Seeded synthetic tensors with the value distributions of the benchmark
configurations (Normal weights with per-row log-uniform sigma, near-one norm
vectors, row-absmax-scaled FP8, MXFP4 / NVFP4 block quantisation), at sizes a
CPU oracle handles in seconds.  Pure numpy/torch on the CPU."""
from __future__ import annotations

import numpy as np
import torch

import oracle

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _bytes(t: torch.Tensor) -> bytes:
    return t.contiguous().view(torch.uint8).numpy().tobytes()


def weights(rows: int, cols: int, seed: int, sigma_rows: bool = True) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g)
    if sigma_rows:
        lo, hi = np.log(0.005), np.log(0.05)
        s = torch.exp(torch.rand(rows, 1, generator=g) * (hi - lo) + lo)
        return w * s
    return w * 0.02


def norm_vector(n: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return 1 + 0.01 * torch.randn(n, generator=g)


def spec_bf16(name, rows, cols, seed, sigma_rows=False):
    return oracle.TensorSpec(name, oracle.DT_BF16, [rows, cols], _bytes(weights(rows, cols, seed, sigma_rows).to(torch.bfloat16)))


def spec_f16(name, rows, cols, seed):
    return oracle.TensorSpec(name, oracle.DT_F16, [rows, cols], _bytes(weights(rows, cols, seed).to(torch.float16)))


def spec_f32(name, rows, cols, seed):
    return oracle.TensorSpec(name, oracle.DT_F32, [rows, cols], _bytes(weights(rows, cols, seed)))


def spec_norm(name, n, seed, dtype=torch.bfloat16, code=None):
    code = code or {torch.bfloat16: oracle.DT_BF16, torch.float16: oracle.DT_F16, torch.float32: oracle.DT_F32}[dtype]
    return oracle.TensorSpec(name, code, [n], _bytes(norm_vector(n, seed).to(dtype)))


def specs_fp8(name, rows, cols, seed):
    w = weights(rows, cols, seed)
    scale = w.abs().amax(dim=1, keepdim=True) / 448.0
    q = (w / scale).to(torch.float8_e4m3fn)
    return [oracle.TensorSpec(name + ".weight", oracle.DT_E4M3, [rows, cols], _bytes(q)),
            oracle.TensorSpec(name + ".weight_scale", oracle.DT_F32, [rows], _bytes(scale.reshape(-1).float()))]


def _quant_e2m1(x: np.ndarray) -> np.ndarray:
    mag = np.abs(x)
    idx = np.abs(mag[..., None] - E2M1).argmin(-1).astype(np.uint8)
    return idx | ((x < 0).astype(np.uint8) << 3)


def _pack_fp4(codes: np.ndarray) -> np.ndarray:
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def specs_mxfp4(name, rows, cols, seed):
    w = weights(rows, cols, seed).numpy().astype(np.float64)
    blk = w.reshape(rows, cols // 32, 32)
    amax = np.maximum(np.abs(blk).max(-1), 1e-30)
    e = np.clip(127 + np.ceil(np.log2(amax / 6.0)), 0, 254).astype(np.uint8)
    scale = np.exp2(e.astype(np.float64) - 127)[..., None]
    packed = _pack_fp4(_quant_e2m1(blk / scale).reshape(rows, cols))
    fp4 = oracle.DT_FP4X2
    return [oracle.TensorSpec(name + "_blocks", fp4, [rows, cols // 2], packed.tobytes(), usage="fp4"),
            oracle.TensorSpec(name + "_scales", oracle.DT_U8, [rows, cols // 32], e.tobytes(), usage="scale")]


def specs_nvfp4(name, rows, cols, seed):
    w = weights(rows, cols, seed).numpy().astype(np.float64)
    g = np.abs(w).max() / (448.0 * 6.0)
    blk = w.reshape(rows, cols // 16, 16)
    amax = np.abs(blk).max(-1)
    s8 = torch.from_numpy(amax / 6.0 / g).to(torch.float32).to(torch.float8_e4m3fn)
    s = s8.to(torch.float32).numpy().astype(np.float64) * g
    s = np.where(s == 0, 1.0, s)[..., None]
    packed = _pack_fp4(_quant_e2m1(blk / s).reshape(rows, cols))
    return [oracle.TensorSpec(name + ".weight", oracle.DT_FP4X2, [rows, cols // 2], packed.tobytes(), usage="fp4"),
            oracle.TensorSpec(name + ".weight_scale", oracle.DT_E4M3, [rows, cols // 16], _bytes(s8), usage="scale"),
            oracle.TensorSpec(name + ".weight_scale_2", oracle.DT_F32, [1], np.array([g], np.float32).tobytes(), usage="global_scale")]


def mixed_model(scale: int = 1):
    """A small state dict touching every layout of the hot path."""
    r, c = 96 * scale, 256 * scale
    specs = [spec_bf16("blk.q.weight", r, c, 1), spec_bf16("blk.k.weight", r // 4, c, 2), spec_f16("blk.o.f16", r, c, 3),
             spec_f32("blk.gate.f32", r, c, 4), spec_norm("blk.norm.weight", c, 5), spec_norm("blk.norm.f32", c, 6, torch.float32),
             spec_norm("scalar.f32", 1, 7, torch.float32)]
    specs += specs_fp8("blk.fp8", r, c, 8) + specs_mxfp4("blk.mx", r, c, 9) + specs_nvfp4("blk.nv", r, c, 10)
    specs.append(oracle.TensorSpec("odd.bf16", oracle.DT_BF16, [4093], _bytes((torch.randn(4093, generator=torch.Generator().manual_seed(11)) * 0.02).to(torch.bfloat16))))
    specs.append(oracle.TensorSpec("empty.f32", oracle.DT_F32, [0, 8], b""))
    specs.append(oracle.TensorSpec("bytes.u8", oracle.DT_U8, [1000], bytes(np.random.default_rng(12).integers(0, 4, 1000, dtype=np.uint8))))
    return specs
