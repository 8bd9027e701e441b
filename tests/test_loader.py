"""Loader-side API: shard planning, the model index, streamed file loads, sharded
directories and the safetensors-shaped accessor.

The CPU cases follow the reference's own tests for these helpers
(tests/ptwm/sharding/test_sharder.py, test_index.py, test_reader.py); the GPU
cases compare every loaded tensor with the oracle's decode of the same file.
"""
import json
import os

import pytest
import torch

import oracle
from _data import mixed_model

import ptwm_b200
from ptwm_b200 import PtwmIndex, plan_shards, read_sharded_ptwm, shard_filename


# ---- host logic ---------------------------------------------------------------
def test_shard_filenames():
    assert shard_filename(1, 7, suffix="ptwm") == "model-00001-of-00007.ptwm"
    assert shard_filename(7, 7, suffix="ptwm") == "model-00007-of-00007.ptwm"
    assert shard_filename(1, 2, suffix="safetensors") == "model-00001-of-00002.safetensors"
    for bad in (0, 8):
        with pytest.raises(ValueError):
            shard_filename(bad, 7, suffix="ptwm")


def test_plan_shards():
    five = [(f"t{i}", 1 << 20) for i in range(5)]
    assert [len(s) for s in plan_shards(five, max_shard_size=2 << 20)] == [2, 2, 1]
    assert len(plan_shards([(f"t{i}", 1 << 10) for i in range(3)], max_shard_size=1 << 30)) == 1
    names = [[n for n, _ in s] for s in plan_shards([("a", 1 << 10), ("big", 4 << 20), ("c", 1 << 10)], max_shard_size=2 << 20)]
    assert names == [["a"], ["big"], ["c"]]
    flat = [n for s in plan_shards(five, max_shard_size=2 << 20) for n, _ in s]
    assert flat == [f"t{i}" for i in range(5)]
    assert plan_shards([], max_shard_size=1) == []
    with pytest.raises(ValueError):
        plan_shards(five, max_shard_size=0)


def test_index_round_trip(tmp_path):
    idx = PtwmIndex(total_size=102538378240, compressed_total_size=56210334752,
                    weight_map={"model.layers.0.q.weight": "model-00001-of-00007.ptwm", "model.layers.99.weight": "model-00007-of-00007.ptwm"})
    p = tmp_path / "model.ptwm.index.json"
    idx.write(p)
    raw = json.loads(p.read_text())
    assert raw["metadata"] == {"total_size": 102538378240, "format": "ptwm", "format_version": 1, "compressed_total_size": 56210334752}
    assert sorted(set(raw["weight_map"].values())) == ["model-00001-of-00007.ptwm", "model-00007-of-00007.ptwm"]
    assert PtwmIndex.read(p) == idx
    bad = tmp_path / "x.json"
    bad.write_text(json.dumps({"metadata": {"format": "other"}, "weight_map": {}}))
    with pytest.raises(ValueError, match="format"):
        PtwmIndex.read(bad)


def test_shell_file_is_plain_safetensors_with_the_container_hash(tmp_path):
    """tests/ptwm/integrations/test_mode_b_shell.py of the reference: the shell opens with stock safetensors, names its
    format and carries the XXH64 of the wrapped bytes as 16 hex digits."""
    xxhash = pytest.importorskip("xxhash")
    from safetensors import safe_open
    blob = oracle.write_container(mixed_model()[:3], chunk_size=4096)
    ptwm_b200.write_mode_b_shell(tmp_path / "shell.safetensors", blob)
    with safe_open(str(tmp_path / "shell.safetensors"), framework="pt") as f:
        assert list(f.keys()) == ["__ptwm_payload__"]
        meta = f.metadata()
        assert meta["weights_format"] == "ptwm-shell" and meta["weights_format_version"] == "1"
        assert meta["ptwm_bytes_xxhash64"] == xxhash.xxh64(blob).hexdigest() and len(meta["ptwm_bytes_xxhash64"]) == 16
        assert f.get_tensor("__ptwm_payload__").numpy().tobytes() == blob


def test_directory_without_a_model_raises(tmp_path):
    with pytest.raises(FileNotFoundError):
        read_sharded_ptwm(tmp_path)


# ---- on the GPU -----------------------------------------------------------------
def _bytes_of(t: torch.Tensor) -> bytes:
    return t.contiguous().view(torch.uint8).cpu().numpy().tobytes()


def _write(path, specs, **options) -> dict:
    blob = oracle.write_container(specs, **options)
    path.write_bytes(blob)
    oc = oracle.Container(blob)
    return {s.name: oc.decode(i) for i, s in enumerate(specs)}


@pytest.mark.gpu
@pytest.mark.parametrize("stream", [dict(), dict(slot_bytes=1 << 16, slots=2, threads=3, pieces=5), dict(slot_bytes=4096, slots=3, threads=1, pieces=1)])
def test_load_file_matches_oracle(tmp_path, stream):
    specs = mixed_model()
    expected = _write(tmp_path / "m.ptwm", specs, chunk_size=8192, emit_crc=True, emit_hash=True, menu=(oracle.HUFFMAN, oracle.RANS, oracle.O1SAC))
    info = {}
    got = ptwm_b200.load_file(tmp_path / "m.ptwm", 0, timings=info, **stream)
    assert list(got) == list(expected)
    for name, raw in expected.items():
        assert _bytes_of(got[name]) == raw, name
    assert info["file_bytes"] > 0 and info["slices"] >= -(-info["file_bytes"] // stream.get("slot_bytes", 128 << 20))
    # a second load reuses the pinned buffers
    again = ptwm_b200.load_file(tmp_path / "m.ptwm", 0, **stream)
    assert all(_bytes_of(again[n]) == raw for n, raw in expected.items())


@pytest.mark.gpu
def test_two_loads_at_once_do_not_share_staging_buffers(tmp_path):
    """Two threads load two different files through small staging sets at the same time; without plane CRCs or hashes a
    slot shared between them would hand one file's bytes to the other unnoticed."""
    import threading
    specs = mixed_model()
    want = [_write(tmp_path / "a.ptwm", specs, chunk_size=4096), _write(tmp_path / "b.ptwm", list(reversed(specs)), chunk_size=2048, menu=(oracle.IDENTITY, oracle.HUFFMAN))]
    got, errors = [None, None], []

    def work(k, path):
        try:
            for _ in range(3):
                got[k] = ptwm_b200.load_file(path, device=0, verify=False, slot_bytes=8192, slots=2, threads=2, pieces=3)
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(0, tmp_path / "a.ptwm")), threading.Thread(target=work, args=(1, tmp_path / "b.ptwm"))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for k in range(2):
        assert {n: _bytes_of(t) for n, t in got[k].items()} == want[k]


@pytest.mark.gpu
def test_load_file_subset_reads_only_its_span(tmp_path):
    specs = mixed_model()
    expected = _write(tmp_path / "m.ptwm", specs, chunk_size=4096)
    names = [specs[3].name, specs[1].name]
    info = {}
    got = ptwm_b200.load_file(tmp_path / "m.ptwm", 0, names=names, timings=info, slot_bytes=1 << 15, slots=2)
    assert sorted(got) == sorted(names)
    assert all(_bytes_of(got[n]) == expected[n] for n in names)
    assert info["file_bytes"] < os.path.getsize(tmp_path / "m.ptwm")
    with pytest.raises(KeyError):
        ptwm_b200.load_file(tmp_path / "m.ptwm", 0, names=["no such tensor"])


@pytest.mark.gpu
def test_load_file_reports_a_truncated_file(tmp_path):
    specs = mixed_model()
    _write(tmp_path / "m.ptwm", specs, chunk_size=4096)
    data = (tmp_path / "m.ptwm").read_bytes()
    (tmp_path / "cut.ptwm").write_bytes(data[:len(data) // 2])
    with pytest.raises((ptwm_b200.PtwmError, ValueError)):
        ptwm_b200.load_file(tmp_path / "cut.ptwm", 0)
    (tmp_path / "empty.ptwm").write_bytes(b"")
    with pytest.raises(ptwm_b200.HeaderParseError):
        ptwm_b200.load_file(tmp_path / "empty.ptwm", 0)


@pytest.mark.gpu
def test_sharded_directory_round_trip(tmp_path):
    specs = mixed_model()
    half = len(specs) // 2
    exp1 = _write(tmp_path / "model-00001-of-00002.ptwm", specs[:half], chunk_size=8192, emit_crc=True)
    exp2 = _write(tmp_path / "model-00002-of-00002.ptwm", specs[half:], forced_codec=oracle.RANS, chunk_size=8192)
    wm = {n: "model-00001-of-00002.ptwm" for n in exp1} | {n: "model-00002-of-00002.ptwm" for n in exp2}
    PtwmIndex(total_size=sum(len(s.raw) for s in specs), compressed_total_size=0, weight_map=wm).write(tmp_path / "model.ptwm.index.json")
    state = read_sharded_ptwm(tmp_path, 0)
    assert set(state) == set(exp1) | set(exp2)
    for name, raw in (exp1 | exp2).items():
        assert _bytes_of(state[name]) == raw, name
    # the same tensor in two shards is an error
    (tmp_path / "model-00002-of-00002.ptwm").write_bytes((tmp_path / "model-00001-of-00002.ptwm").read_bytes())
    with pytest.raises(ValueError, match="multiple shards"):
        read_sharded_ptwm(tmp_path, 0)


@pytest.mark.gpu
def test_single_file_directory_and_device_writer(tmp_path):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(5)
    tensors = {"a.weight": (torch.randn(300, 257, generator=g) * 0.02).to(torch.bfloat16).to(dev),
               "b.weight": torch.randn(129, 64, generator=g).to(dev),
               "c.bytes": torch.randint(0, 255, (1000,), generator=g, dtype=torch.uint8).to(dev)}
    one = tmp_path / "one"
    idx = ptwm_b200.save_sharded(tensors, one, config=ptwm_b200.CompressionConfig(streaming_chunk=4096))
    assert sorted(os.listdir(one)) == ["model.ptwm"] and set(idx.weight_map.values()) == {"model.ptwm"}
    state = read_sharded_ptwm(one, 0)
    assert all(torch.equal(state[n], t) for n, t in tensors.items())
    many = tmp_path / "many"
    idx = ptwm_b200.save_sharded(tensors, many, max_shard_size=20_000, config=ptwm_b200.CompressionConfig(streaming_chunk=4096))
    assert sorted(os.listdir(many)) == ["model-00001-of-00003.ptwm", "model-00002-of-00003.ptwm", "model-00003-of-00003.ptwm", "model.ptwm.index.json"]
    assert PtwmIndex.read(many / "model.ptwm.index.json") == idx
    assert idx.total_size == sum(t.numel() * t.element_size() for t in tensors.values())
    state = read_sharded_ptwm(many, 0)
    assert list(state) == list(tensors) and all(torch.equal(state[n], t) for n, t in tensors.items())


@pytest.mark.gpu
def test_safe_open_modes(tmp_path):
    from safetensors.torch import save_file
    specs = mixed_model()
    expected = _write(tmp_path / "model.ptwm", specs, chunk_size=8192, emit_crc=True)
    # mode A: a .ptwm file
    with ptwm_b200.SafeOpen(str(tmp_path / "model.ptwm"), framework="pt", device="cuda:0") as f:
        assert f.keys() == list(expected) and f.metadata() is None
        for name, raw in expected.items():
            assert _bytes_of(f.get_tensor(name)) == raw
        with pytest.raises(NotImplementedError):
            f.get_slice(specs[0].name)
        with pytest.raises(KeyError):
            f.get_tensor("no such tensor")
        with pytest.raises(AttributeError):
            f.no_such_attribute
    # mode B: the container wrapped as one tensor of a safetensors file
    ptwm_b200.write_mode_b_shell(tmp_path / "shell.safetensors", (tmp_path / "model.ptwm").read_bytes())
    with ptwm_b200.SafeOpen(str(tmp_path / "shell.safetensors"), framework="pt", device="cuda:0") as f:
        assert f.keys() == list(expected) and f.metadata()["weights_format"] == "ptwm-shell"
        assert all(_bytes_of(f.get_tensor(n)) == raw for n, raw in expected.items())
    # anything else goes to the safetensors library untouched
    plain = {"x": torch.arange(12, dtype=torch.float32).reshape(3, 4)}
    save_file(plain, str(tmp_path / "plain.safetensors"))
    with ptwm_b200.SafeOpen(str(tmp_path / "plain.safetensors"), framework="pt", device="cpu") as f:
        assert list(f.keys()) == ["x"] and torch.equal(f.get_tensor("x"), plain["x"])
        assert f.get_slice("x")[1:2].shape == (1, 4)


@pytest.mark.gpu
def test_tensor_index_opens_files_in_place(tmp_path):
    specs = mixed_model()
    expected = _write(tmp_path / "m.ptwm", specs, chunk_size=8192)
    idx = ptwm_b200.TensorIndex.open(tmp_path / "m.ptwm", device=0)
    assert idx.layout == "compact" and idx.names() == list(expected) and len(idx) == len(expected)
    for name, tensor in idx.stream_tensors([specs[2].name, specs[0].name]):
        assert _bytes_of(tensor) == expected[name]
    assert idx.get_bytes(specs[1].name) == expected[specs[1].name]
    assert [e.name for e in idx.entries()] == idx.names() and idx.entry(specs[0].name) == ptwm_b200.TensorEntry(specs[0].name)
    with pytest.raises(KeyError):
        idx.entry("absent")
    (tmp_path / "junk.ptwm").write_bytes(b"not a container at all")
    with pytest.raises(ValueError):
        ptwm_b200.TensorIndex(tmp_path / "junk.ptwm")
