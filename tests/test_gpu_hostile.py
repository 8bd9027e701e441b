"""Damaged payloads must end in an error code (or different bytes), never in a
fault: every decode loop is bounded by the symbol count and every read is
clamped to the resident blob.  Mirrors the reference's accepted outcomes
(tests/ptwm/core/test_decompressor_errors.py:35-77)."""
import numpy as np
import pytest
import torch

import oracle
import ptwm_b200
from _data import spec_bf16, specs_fp8

pytestmark = pytest.mark.gpu


def _raw(t):
    return t.contiguous().view(torch.uint8).cpu().numpy().tobytes()


@pytest.mark.parametrize("codec", [oracle.HUFFMAN, oracle.RANS, oracle.TANS])
def test_mutated_payload_bytes(codec):
    specs = [spec_bf16("w", 64, 512, 3)] + specs_fp8("f", 32, 256, 4)
    blob = oracle.write_container(specs, forced_codec=codec, chunk_size=4096)
    base = ptwm_b200.ContainerHandle(blob, device=0, verify=False)
    infos = base.tensor_infos()
    rng = np.random.default_rng(5)
    outcomes = {"error": 0, "different": 0, "same": 0}
    for trial in range(40):
        t = infos[int(rng.integers(0, len(infos)))]
        pos = int(rng.integers(t["first_byte"], t["end_byte"]))
        m = bytearray(blob)
        m[pos] ^= int(rng.integers(1, 256))
        try:
            h = ptwm_b200.ContainerHandle(bytes(m), device=0, verify=False)
            got = dict(h.decode_model())
        except (ptwm_b200.PtwmError, ValueError):
            outcomes["error"] += 1
            continue
        same = all(_raw(got[s.name]) == s.raw for s in specs)
        outcomes["same" if same else "different"] += 1
    assert outcomes["error"] + outcomes["different"] > 0
    # the context is still usable afterwards
    assert _raw(dict(base.decode_model())["w"]) == specs[0].raw


def test_truncated_container_is_refused():
    specs = [spec_bf16("w", 32, 256, 6)]
    blob = oracle.write_container(specs, chunk_size=2048)
    for cut in (10, len(blob) // 2, len(blob) - 1):
        with pytest.raises((ptwm_b200.PtwmError, ValueError)):
            ptwm_b200.ContainerHandle(blob[:cut], device=0)
