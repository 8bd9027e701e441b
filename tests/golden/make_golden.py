"""Regenerates the committed golden containers under tests/golden/oracle/.

Each case is a small seeded model written by the CPU oracle's writer
(oracle.write_container / write_compact, which restate the reference's
compressor.rs framing) together with the concatenated raw tensor bytes it must
decode to.  Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from _data import mixed_model  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "oracle")
CASES = {
    "mixed_whole": dict(),
    "mixed_chunk4k_crc": dict(chunk_size=4096, emit_crc=True),
    "mixed_chunk1000_hash_crc": dict(chunk_size=1000, emit_hash=True, emit_crc=True),
    "mixed_huffman_chunk8k": dict(forced_codec=oracle.HUFFMAN, chunk_size=8192, emit_crc=True),
    "mixed_rans_chunk8k": dict(forced_codec=oracle.RANS, chunk_size=8192, emit_hash=True),
    "mixed_tans_chunk8k": dict(forced_codec=oracle.TANS, chunk_size=8192),
    "mixed_menu_huff_rans_o1sac": dict(menu=(oracle.HUFFMAN, oracle.RANS, oracle.O1SAC), emit_crc=True, emit_hash=True),
}


def main():
    os.makedirs(OUT, exist_ok=True)
    specs = mixed_model()
    manifest = {}
    for name, kw in CASES.items():
        blob = oracle.write_container(specs, **kw)
        c = oracle.Container(blob)
        for i, s in enumerate(specs):
            assert c.decode(i) == s.raw, (name, s.name)
        with open(os.path.join(OUT, name + ".ptwm"), "wb") as f:
            f.write(blob)
        manifest[name] = {"bytes": len(blob), "tensors": {s.name: [len(s.raw), hashlib.sha256(s.raw).hexdigest()] for s in specs}}
    frames = {}
    for s in specs[:8]:
        for tag, kw in (("bare", {}), ("hash", dict(emit_hash=True)), ("crc", dict(emit_crc=True))):
            blob = oracle.write_compact(s, **kw)
            fn = f"frame_{s.name}_{tag}.ptws"
            with open(os.path.join(OUT, fn), "wb") as f:
                f.write(blob)
            frames[fn] = [len(s.raw), hashlib.sha256(s.raw).hexdigest()]
    manifest["frames"] = frames
    with open(os.path.join(OUT, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print("wrote", len(CASES), "containers and", len(frames), "frames to", OUT)


if __name__ == "__main__":
    main()
