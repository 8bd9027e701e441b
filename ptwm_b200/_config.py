"""Configuration and errors of the decode API; mirrors the reference's
``python/ptwm/_config.py:260-274`` and ``python/ptwm/_exceptions.py``."""
from __future__ import annotations

from dataclasses import dataclass


class HeaderParseError(ValueError):
    """The blob is too short or does not start with a known magic."""


class InvalidDTypeError(TypeError):
    """The record's dtype code has no torch dtype."""


@dataclass(frozen=True, kw_only=True)
class DecompressionConfig:
    """Same fields as the reference's ``DecompressionConfig``.  ``device`` is
    the CUDA ordinal the tensors are decoded on and returned from; the
    reference rejects any value (``core/_decompressor.py:69-77``), here it
    defaults to the current CUDA device.  ``verify`` adds the integrity checks
    the container carries (plane CRC-32, XXH64 payload hash), which the
    reference always runs."""
    threads: int | None = None
    delta_second_data: bytes | None = None
    skip_missing: bool = False
    codec: str | None = None
    device: int | None = None
    verify: bool = True
