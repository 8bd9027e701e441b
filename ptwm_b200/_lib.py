"""ctypes binding of ``libptwm_b200.so`` (declared in ``include/ptwm_b200.h``).

The library holds every CUDA kernel of the package.  There is no fallback: if
it is missing or cannot be loaded, importing the decode/encode entry points
fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PTWM_B200_LIB") or os.path.join(_HERE, "libptwm_b200.so")  # PTWM_B200_LIB: load another build of the same library
_SOURCES = [os.path.join(_HERE, "csrc", f) for f in ("unity.cu", "ptwm_b200.cu", "encoder.cu", "kernels.cuh", "encode.cuh", "encode_tables.cuh", "noalloc.cu",
                                                      "format.hpp", "host_common.hpp", "plan.h")] + [
    os.path.join(_HERE, "..", "include", "ptwm_b200.h")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread", "-shared"]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA library for sm_100a in-tree with nvcc."""
    srcs = [s for s in _SOURCES if os.path.exists(s)]
    stale = force or not os.path.exists(LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in srcs)
    if stale:
        nvcc = os.environ.get("NVCC", "nvcc")
        cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, os.path.join(_HERE, "csrc", "unity.cu")]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        if verbose:
            print(res.stderr)
    return LIB_PATH


class TensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype_name", C.c_char_p), ("dtype_code", C.c_uint16), ("ndim", C.c_uint8), ("has_shape", C.c_uint8),
                ("has_hash", C.c_uint8), ("has_crc", C.c_uint8), ("supported", C.c_uint8), ("kind", C.c_uint8), ("shape", C.c_uint64 * 8),
                ("orig_size", C.c_uint64), ("compressed", C.c_uint64), ("first_byte", C.c_uint64), ("end_byte", C.c_uint64),
                ("unsupported_reason", C.c_char_p)]


class EncodeTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dev_ptr", C.c_uint64), ("nbytes", C.c_uint64), ("shape", C.c_uint64 * 8), ("dtype_code", C.c_uint16),
                ("ndim", C.c_uint8), ("usage", C.c_uint8), ("post_op", C.c_uint8), ("post_plane", C.c_uint8), ("post_k", C.c_uint8), ("reserved_", C.c_uint8)]


class EncodeOptions(C.Structure):
    _fields_ = [("chunk_size", C.c_uint32), ("menu", C.c_uint32), ("forced_codec", C.c_int32), ("emit_plane_crc", C.c_uint8),
                ("emit_payload_hash", C.c_uint8), ("candidates", C.c_uint8), ("reserved", C.c_uint8 * 1)]


_SIGNATURES = {
    "ptwm_b200_encode_model": (C.c_int64, [C.POINTER(EncodeTensor), C.c_size_t, C.POINTER(EncodeOptions), C.c_uint32, C.c_uint64, C.POINTER(C.c_void_p)]),
    "ptwm_b200_encoded_size": (C.c_uint64, [C.c_void_p]),
    "ptwm_b200_encoded_device_ptr": (C.c_uint64, [C.c_void_p]),
    "ptwm_b200_encoded_copy": (C.c_int64, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "ptwm_b200_encoded_copy_to_device": (C.c_int64, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64]),
    "ptwm_b200_encoded_plane_codec": (C.c_int32, [C.c_void_p, C.c_size_t, C.c_size_t]),
    "ptwm_b200_encoded_free": (None, [C.c_void_p]),
    "ptwm_b200_last_error": (C.c_char_p, []),
    "ptwm_b200_blake3": (None, [C.c_char_p, C.c_size_t, C.c_char_p]),
    "ptwm_b200_xxh64": (C.c_uint64, [C.c_char_p, C.c_size_t]),
    "ptwm_b200_open": (C.c_int64, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "ptwm_b200_open_shard": (C.c_int64, [C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]),
    "ptwm_b200_close": (None, [C.c_void_p]),
    "ptwm_b200_tensor_count": (C.c_size_t, [C.c_void_p]),
    "ptwm_b200_tensor_info_get": (C.c_int64, [C.c_void_p, C.c_size_t, C.POINTER(TensorInfo)]),
    "ptwm_b200_plan_create": (C.c_int64, [C.c_void_p, C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_void_p)]),
    "ptwm_b200_plan_destroy": (None, [C.c_void_p]),
    "ptwm_b200_plan_out_bytes": (C.c_uint64, [C.c_void_p]),
    "ptwm_b200_plan_scratch_bytes": (C.c_uint64, [C.c_void_p]),
    "ptwm_b200_plan_out_offset": (C.c_uint64, [C.c_void_p, C.c_size_t]),
    "ptwm_b200_plan_blob_span": (None, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "ptwm_b200_plan_stats": (None, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]),
    "ptwm_b200_plan_run": (C.c_int64, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32,
                                       C.c_uint32, C.c_uint64]),
    "ptwm_b200_plan_finish": (C.c_int64, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64]),
    "ptwm_b200_plan_prepare": (C.c_int64, [C.c_void_p, C.c_uint32]),
    "ptwm_b200_plan_device_bytes": (C.c_uint64, [C.c_void_p]),
    "ptwm_b200_plan_prepare_in": (C.c_int64, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint64]),
    "ptwm_b200_plan_timings": (C.c_int64, [C.c_void_p, C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]),
    "ptwm_b200_decode_plane_noalloc": (C.c_int64, [C.c_uint8, C.c_void_p, C.c_size_t, C.c_char_p, C.c_size_t, C.c_uint64, C.c_size_t, C.c_uint64,
                                                   C.c_size_t, C.c_uint32, C.c_uint64]),
    "ptwm_b200_crc32_by_runs": (C.c_uint32, [C.c_char_p, C.c_size_t, C.c_size_t]),
    "ptwm_b200_fit_shared_states_host": (C.c_int64, [C.POINTER(C.c_char_p), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.c_size_t, C.c_void_p, C.c_size_t,
                                                     C.POINTER(C.c_uint32)]),
    "ptwm_hardware_backend_v1_cuda_stream_handle": (C.c_uint64, [C.c_uint32]),
    "ptwm_plane_codec_v1_cuda_stream_handle": (C.c_uint64, [C.c_uint32]),
    "ptwm_hardware_backend_v1_dispatch_decode_cuda": (C.c_int64, [C.c_uint8, C.c_void_p, C.c_size_t, C.c_char_p, C.c_size_t, C.c_uint64, C.c_size_t,
                                                                  C.c_uint64, C.c_size_t, C.c_uint32]),
    "ptwm_plane_codec_v1_decode_cuda": (C.c_int64, [C.c_uint8, C.c_void_p, C.c_size_t, C.c_char_p, C.c_size_t, C.c_uint64, C.c_size_t, C.c_uint64,
                                                    C.c_size_t, C.c_uint32]),
    "ptwm_plane_codec_v1_encode_cuda": (C.c_int64, [C.c_uint8, C.c_void_p, C.c_size_t, C.c_char_p, C.c_size_t, C.c_uint64, C.c_size_t, C.c_uint64,
                                                    C.c_size_t, C.POINTER(C.c_uint64), C.c_uint32]),
    "ptwm_plane_codec_v1_encode": (C.c_int64, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "ptwm_plane_codec_v1_decode": (C.c_int64, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "ptwm_plane_codec_v1_decode_stateful": (C.c_int64, [C.c_uint8, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: the CUDA kernels are not built. Run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(needs nvcc); ptwm_b200 has no CPU fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().ptwm_b200_last_error().decode("utf-8", "replace")


def fit_shared_states_host(planes, row_lens) -> list[bytes]:
    """The encoder's shared Order1ScaleAC states for these planes (bytes objects, rows of row_lens[k]), fitted on the host."""
    n = len(planes)
    arr = (C.c_char_p * n)(*[bytes(p) for p in planes])
    lens = (C.c_uint64 * n)(*[len(p) for p in planes])
    rows = (C.c_uint32 * n)(*[int(r) for r in row_lens])
    cap = 8 * (32 + 512 + 512 * 256)
    out = C.create_string_buffer(cap)
    state_lens = (C.c_uint32 * 8)()
    k = lib().ptwm_b200_fit_shared_states_host(arr, lens, rows, n, out, cap, state_lens)
    if k < 0:
        raise RuntimeError(last_error())
    states, pos = [], 0
    for i in range(k):
        states.append(out.raw[pos:pos + state_lens[i]])
        pos += state_lens[i]
    return states


def xxh64(data: bytes) -> int:
    """XXH64 (seed 0) of host bytes, computed by the library's host code."""
    return int(lib().ptwm_b200_xxh64(data, len(data)))
