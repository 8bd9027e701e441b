"""The benchmark configurations at their stated sizes.

Tensors of the shapes and value distributions the reference's configurations name (fp32 and fp16 transformer block sets
with per-row sigma, FP8-E4M3 weights with fp32 row scales, MXFP4 / NVFP4 layers with their block scales) are generated on
the GPU from fixed seeds, written by the device encoder with plane CRC-32s and XXH64 payload hashes, and decoded with
both checks on.  Checks that do not depend on the size:

* every decoded tensor equals its source bit for bit (torch.equal on the bytes);
* the container verifies itself (a wrong plane fails its CRC, a wrong tensor its hash);
* the CPU oracle, a restatement of the reference decoder, decodes the device-written container to the same bytes
  (all of it where that takes seconds, a sample of the tensors otherwise);
* the device-written container is within 1 % of the oracle writer's size on that sample.
"""
import numpy as np
import pytest
import torch

import oracle
import ptwm_b200
from ptwm_b200.compressor import CompressionConfig, ORDER1_SCALE_AC, compress_model

pytestmark = pytest.mark.gpu

_CODE = {torch.float32: oracle.DT_F32, torch.float16: oracle.DT_F16, torch.bfloat16: oracle.DT_BF16, torch.float8_e4m3fn: oracle.DT_E4M3, torch.uint8: oracle.DT_U8}


def _weights(rows, cols, seed):
    """Normal(0, sigma_row), sigma_row log-uniform in [0.005, 0.05] per row."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, cols, generator=g, device="cuda")
    lo, hi = np.log(0.005), np.log(0.05)
    return w * torch.exp(torch.rand(rows, 1, generator=g, device="cuda") * (hi - lo) + lo)


def _norm(n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return 1 + 0.01 * torch.randn(n, generator=g, device="cuda")


def _block_set(dtype):
    d, ffn = 4096, 14336
    shapes = [("q", d, d), ("k", d, d), ("v", d, d), ("o", d, d), ("gate", ffn, d), ("up", ffn, d), ("down", d, ffn)]
    tensors = {f"blk.{n}_proj.weight": _weights(r, c, 1000 + i).to(dtype) for i, (n, r, c) in enumerate(shapes)}
    tensors["blk.input_layernorm.weight"] = _norm(d, 1100).to(dtype)
    tensors["blk.post_attention_layernorm.weight"] = _norm(d, 1101).to(dtype)
    return tensors


def _bytes(t):
    return t.contiguous().view(torch.uint8).reshape(-1)


def _spec(name, t, usage="standard"):
    code = oracle.DT_U8 if usage == "fp4" else _CODE[t.dtype]
    return oracle.TensorSpec(name, code, list(t.shape), _bytes(t).cpu().numpy().tobytes(), usage=usage)


def _round_trip(tensors, usage, cfg, oracle_names, size_names=()):
    enc = compress_model(tensors, cfg, usage=usage)
    blob = enc.to_bytes()
    h = ptwm_b200.ContainerHandle(blob, device=0, verify=True)
    got = dict(h.decode_model())
    assert list(got) == list(tensors)
    for name, t in tensors.items():
        assert torch.equal(_bytes(got[name]), _bytes(t)), name
    del got
    oc = oracle.Container(blob)
    names = list(tensors)
    for name in oracle_names:
        assert oc.decode(names.index(name)) == _bytes(tensors[name]).cpu().numpy().tobytes(), name
    if size_names:
        sub = {n: tensors[n] for n in size_names}
        ours = compress_model(sub, cfg, usage={n: u for n, u in usage.items() if n in sub}).size
        specs = [_spec(n, t, usage.get(n, "standard")) for n, t in sub.items()]
        theirs = len(oracle.write_container(specs, chunk_size=cfg.streaming_chunk, menu=tuple(cfg.codec_menu), emit_crc=cfg.emit_plane_crc, emit_hash=cfg.emit_payload_hash))
        assert abs(ours - theirs) <= 0.01 * theirs, (ours, theirs)
    return enc


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_transformer_block_set(dtype):
    """fp32: the four-plane path (three mantissa planes, one exponent plane); fp16: the two-plane path with the 16-bit reorder."""
    tensors = _block_set(dtype)
    assert sum(t.numel() * t.element_size() for t in tensors.values()) == (973_111_296 if dtype == torch.float32 else 486_555_648)
    cfg = CompressionConfig(streaming_chunk=65536, emit_plane_crc=True, emit_payload_hash=True)
    _round_trip(tensors, {}, cfg, oracle_names=["blk.k_proj.weight", "blk.input_layernorm.weight"], size_names=["blk.k_proj.weight", "blk.post_attention_layernorm.weight"])


def test_fp8_weights_with_row_scales():
    tensors = {}
    for i, (rows, cols) in enumerate([(14336, 4096), (4096, 14336)]):
        w = _weights(rows, cols, 2000 + i)
        scale = w.abs().amax(dim=1, keepdim=True) / 448.0
        tensors[f"l{i}.weight"] = (w / scale).to(torch.float8_e4m3fn)
        tensors[f"l{i}.weight_scale"] = scale.reshape(-1).float()
    cfg = CompressionConfig(streaming_chunk=65536, emit_plane_crc=True, emit_payload_hash=True)
    _round_trip(tensors, {}, cfg, oracle_names=list(tensors), size_names=["l1.weight", "l1.weight_scale"])


def _e2m1_codes(x):
    levels = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=x.device)
    idx = (x.abs().unsqueeze(-1) - levels).abs().argmin(-1).to(torch.uint8)
    return idx | ((x < 0).to(torch.uint8) << 3)


def _pack(codes):
    return codes[..., 0::2] | (codes[..., 1::2] << 4)


def test_microscaling_layers_use_the_scale_coder():
    rows, cols = 14336, 4096
    w = _weights(rows, cols, 3000).double()
    # MXFP4: blocks of 32, E8M0 scales
    blk = w.reshape(rows, cols // 32, 32)
    amax = blk.abs().amax(-1).clamp_min(1e-30)
    e = (127 + torch.ceil(torch.log2(amax / 6.0))).clamp(0, 254).to(torch.uint8)
    mx = _pack(_e2m1_codes((blk / torch.exp2(e.double() - 127).unsqueeze(-1)).reshape(rows, cols).float()))
    # NVFP4: blocks of 16, E4M3 scales, one fp32 scale for the tensor
    g = w.abs().max() / (448.0 * 6.0)
    blk = w.reshape(rows, cols // 16, 16)
    s8 = (blk.abs().amax(-1) / 6.0 / g).float().to(torch.float8_e4m3fn)
    s = s8.float().double() * g
    s = torch.where(s == 0, torch.ones_like(s), s).unsqueeze(-1)
    nv = _pack(_e2m1_codes((blk / s).reshape(rows, cols).float()))
    tensors = {"mx.blocks": mx.contiguous(), "mx.scales": e.contiguous(), "nv.weight": nv.contiguous(), "nv.weight_scale": s8.contiguous(),
               "nv.weight_scale_2": g.float().reshape(1)}
    assert tensors["mx.blocks"].shape == (14336, 2048) and tensors["mx.scales"].shape == (14336, 128) and tensors["nv.weight_scale"].shape == (14336, 256)
    usage = {"mx.blocks": "fp4", "mx.scales": "scale", "nv.weight": "fp4", "nv.weight_scale": "scale", "nv.weight_scale_2": "global_scale"}
    cfg = CompressionConfig(streaming_chunk=65536, emit_plane_crc=True, emit_payload_hash=True)
    enc = _round_trip(tensors, usage, cfg, oracle_names=list(tensors), size_names=["mx.scales", "nv.weight_scale", "nv.weight_scale_2"])
    assert enc.plane_codecs["mx.scales"] == [ORDER1_SCALE_AC] and enc.plane_codecs["nv.weight_scale"] == [ORDER1_SCALE_AC], enc.plane_codecs
