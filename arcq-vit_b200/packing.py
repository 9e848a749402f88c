"""Host-side bit packing of ARCQ codes: the on-disk layout of the packed checkpoint.

Code j of a row occupies bits [j*bits, (j+1)*bits) of the row's little-endian bit
stream, least significant bit first in each byte, rows padded to whole bytes --
the layout of the reference's ``pack_codes_py`` / ``unpack_codes_py``
(methods/fair_qat_framework/fair_qat/arcq_packed_py.py:8-78), which loop over columns in
Python; these are vectorised with numpy's bit packing.  CUDA tensors go through the
device kernels instead.
"""
from __future__ import annotations

import numpy as np
import torch


def _check_bits(bits: int) -> None:
    if bits not in (2, 3, 4):
        raise ValueError(f"bits must be 2/3/4, got {bits}")


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """integer codes [R, length] -> uint8 [R, ceil(length*bits/8)]."""
    _check_bits(bits)
    if codes.dim() != 2:
        raise ValueError(f"codes must be 2D, got {codes.dim()}")
    if codes.is_cuda:
        from . import ops
        return ops.pack_codes(codes, bits)
    c = codes.detach().numpy().astype(np.uint8) & np.uint8((1 << bits) - 1)
    R, length = c.shape
    planes = (c[:, :, None] >> np.arange(bits, dtype=np.uint8)) & np.uint8(1)      # [R, length, bits], LSB first
    stream = planes.reshape(R, length * bits)
    packed = np.packbits(stream, axis=1, bitorder="little")                      # pads each row to whole bytes
    return torch.from_numpy(np.ascontiguousarray(packed))


def unpack_codes_u8(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    """uint8 [R, ceil(length*bits/8)] -> uint8 [R, length]."""
    _check_bits(bits)
    if packed.is_cuda:
        from . import ops
        return ops.unpack_codes_u8(packed, bits, length)
    p = packed.detach().numpy().astype(np.uint8)
    R = p.shape[0]
    stream = np.unpackbits(p, axis=1, bitorder="little")[:, : length * bits].reshape(R, length, bits)
    codes = (stream << np.arange(bits, dtype=np.uint8)).sum(axis=2).astype(np.uint8)
    return torch.from_numpy(np.ascontiguousarray(codes))


def unpack_codes(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    """As ``unpack_codes_u8`` but int64, like the reference's ``unpack_codes_py``."""
    return unpack_codes_u8(packed, bits, length).to(torch.int64)
