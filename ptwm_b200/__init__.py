"""ptwm_b200 — decode (and encode) of ptwm containers on NVIDIA B200.

The package is a thin Python layer over ``libptwm_b200.so`` (CUDA kernels for
sm_100a plus the host container parser and planner).  See
``include/ptwm_b200.h`` for the C ABI.
"""
from ._config import DecompressionConfig, HeaderParseError, InvalidDTypeError
from ._lib import EXPORTED_SYMBOLS, LIB_PATH, build
from .compressor import CompressionConfig, EncodedContainer, compress_model
from .loader import PtwmIndex, SafeOpen, load_file, plan_shards, read_sharded_ptwm, save_sharded, shard_filename, write_mode_b_shell
from .container import NO_SYNC, TIME_KERNELS, VERIFY_CRC, VERIFY_HASH, ContainerHandle, DecodePlan, Decompressor, PtwmError, TensorEntry, TensorIndex

__all__ = ["CompressionConfig", "EncodedContainer", "compress_model", "DecompressionConfig", "HeaderParseError", "InvalidDTypeError", "EXPORTED_SYMBOLS", "LIB_PATH", "build", "ContainerHandle",
           "DecodePlan", "Decompressor", "PtwmError", "TensorEntry", "TensorIndex", "PtwmIndex", "SafeOpen", "load_file", "plan_shards", "read_sharded_ptwm", "save_sharded",
           "shard_filename", "write_mode_b_shell", "VERIFY_CRC", "VERIFY_HASH", "NO_SYNC", "TIME_KERNELS"]
