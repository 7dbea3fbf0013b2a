"""FragPack KV page records: format constants, tables and the record codec.

API-compatible with the reference ``fragpack/compression/attn_page.py`` (same
names, arguments, return types and byte format, documented there at :1-44).
The difference is where the work runs: with a CUDA device
:func:`encode_record` and :func:`decode_record` call the sm_100a kernels
through the C ABI (``fp_encode_records`` / ``fp_decode_records``); without one
they use the numpy codec of :mod:`fragpack_b200.compression.host_codec`, which
gives the same bytes, so that offline tools and calibration machines work as
they do with the reference.  (Only this offline package has a host form; the
operators in ``fragpack_b200.ops`` have none.)  Calibration and the LUT
builders are small host-side table manipulations and stay in numpy, as in the
reference (they run offline or once at start-up).

Record layout in brief (one record = 128 tokens x 128 dims BF16 of one layer,
K-or-V and KV head, permuted into the order of ``mma.m16n8k16`` A fragments):

* ``[0, 16384)`` low bytes, thread chunk ``j`` of owner ``t`` at ``16 (256 j + t)``;
* ``[16384, 22528)`` 3-bit primary codes, three u32 per 32 scalars;
* a variable region (48-byte header, escape nibbles, raw list) of 48..2048
  bytes in 16-byte steps;
* or, when that does not fit, the raw 32768-byte record in fragment order.
"""

from __future__ import annotations

import struct

import numpy as np
from numpy.typing import NDArray

PAGE_TOKENS = 128
HEAD_DIM = 128
RECORD_SCALARS = PAGE_TOKENS * HEAD_DIM
GROUP_SCALARS = 32
WARP_SCALARS = 2048
WARPS = RECORD_SCALARS // WARP_SCALARS
PRIMARY_DIRECT = 7
EXTENDED = 15
TABLE_ENTRIES = PRIMARY_DIRECT + EXTENDED
RAW_NIBBLE = 15
HEADER_BYTES = 48
LOW_BYTES = RECORD_SCALARS
SYMBOL_BYTES = RECORD_SCALARS * 3 // 8
DENSE_BYTES = LOW_BYTES + SYMBOL_BYTES
VAR_CAP = 2048
THREADS = 256
LOW_CHUNKS = 4
SYMBOL_CHUNKS = 3
WORDS = 8
RAW_RECORD_BYTES = RECORD_SCALARS * 2
MAX_WARP_RAW = 32
# Block blob (reference attn_page.py:72-78).
BLOB_MAGIC = 0x424B5046  # "FPKB"
BLOB_FIXED_BYTES = 64
BLOB_ALIGN = 4096


def calibrate_table(high_bytes: NDArray[np.uint8]) -> NDArray[np.uint8]:
    """Pick the 22 most frequent high bytes of one (layer, kv, head).

    Reference: ``attn_page.py:97-111``.  Ties go to the smaller byte value.

    Args:
        high_bytes: Calibration high bytes of any shape.

    Returns:
        uint8 array of ``TABLE_ENTRIES`` bytes, most frequent first.
    """
    counts = np.bincount(np.asarray(high_bytes, dtype=np.uint8).ravel(), minlength=256)
    # Sort key: descending count, then ascending byte value.
    order = np.lexsort((np.arange(256), -counts))
    return order[:TABLE_ENTRIES].astype(np.uint8)


def rank_table(table: NDArray[np.uint8]) -> NDArray[np.uint8]:
    """``rank_of[256]``: table position of each high byte, 255 when absent."""
    rank_of = np.full(256, 255, dtype=np.uint8)
    rank_of[np.asarray(table, dtype=np.uint8)] = np.arange(TABLE_ENTRIES, dtype=np.uint8)
    return rank_of


def primary_lut(table: NDArray[np.uint8]) -> tuple[int, int]:
    """Two little-endian u32 words of the 8-byte primary ``prmt`` table.

    Reference: ``attn_page.py:114-128``; byte 7 (the escape code) is zero.
    """
    entries = bytes(np.asarray(table[:PRIMARY_DIRECT], dtype=np.uint8)) + b"\x00"
    lo, hi = struct.unpack("<II", entries)
    return lo, hi


def secondary_lut(table: NDArray[np.uint8]) -> bytes:
    """The 16-byte extended table indexed by escape nibble (entries 7-21, then 0).

    Reference: ``attn_page.py:131-143``.
    """
    return bytes(np.asarray(table[PRIMARY_DIRECT:TABLE_ENTRIES], dtype=np.uint8)) + b"\x00"


def _device_luts(table: NDArray[np.uint8]):
    import torch

    dev = torch.device("cuda", torch.cuda.current_device())
    plut = torch.from_numpy(np.array(primary_lut(table), np.uint32).view(np.int32)).to(dev)
    slut = torch.from_numpy(np.frombuffer(secondary_lut(table), np.uint8).copy()).to(dev)
    return plut, slut


def encode_record(raw: NDArray[np.uint16], table: NDArray[np.uint8], kv: int) -> bytes:
    """Encode one token-major ``[PAGE_TOKENS, HEAD_DIM]`` BF16 record (on the GPU when there is one).

    Reference: ``attn_page.py:146-209``; the bytes are identical.

    Args:
        raw: BF16 bit patterns as uint16.
        table: Head table from :func:`calibrate_table`.
        kv: 0 for a K record, 1 for a V record.

    Returns:
        Record bytes: coded, or the ``RAW_RECORD_BYTES`` raw fallback.

    Raises:
        ValueError: If ``raw`` has the wrong size.
        RuntimeError: If a CUDA device is present but the kernel library is not built.
    """
    import torch

    values = np.ascontiguousarray(raw, dtype=np.uint16).reshape(-1)
    if values.size != RECORD_SCALARS:
        raise ValueError("record must hold PAGE_TOKENS * HEAD_DIM scalars")
    if not torch.cuda.is_available():
        from fragpack_b200.compression import host_codec

        return host_codec.encode(values, rank_table(table), int(kv))
    from fragpack_b200.ops.fragpack_ext import check, extension, stream_ptr

    dev = torch.device("cuda", torch.cuda.current_device())
    src = torch.from_numpy(values.view(np.int16).copy()).to(dev)
    rank_of = torch.from_numpy(rank_table(table)).to(dev)
    which = torch.tensor([int(kv)], dtype=torch.int32, device=dev)
    out = torch.empty(RAW_RECORD_BYTES, dtype=torch.uint8, device=dev)
    length = torch.empty(1, dtype=torch.int32, device=dev)
    check(
        extension().fp_encode_records(
            src.data_ptr(), 1, rank_of.data_ptr(), None, which.data_ptr(), out.data_ptr(),
            RAW_RECORD_BYTES, length.data_ptr(), stream_ptr(),
        )
    )
    n = int(length.item())
    return out[:n].cpu().numpy().tobytes()


def decode_record(record: bytes, table: NDArray[np.uint8], kv: int) -> NDArray[np.uint16]:
    """Decode one record, on the GPU when there is one (reference ``attn_page.py:212-269``).

    Args:
        record: Encoded record.
        table: Head table used to encode it.
        kv: The ``kv`` the record was encoded with.

    Returns:
        uint16 ``[PAGE_TOKENS, HEAD_DIM]`` BF16 bit patterns.

    Raises:
        ValueError: If the length is not a possible record length.
        RuntimeError: If a CUDA device is present but the kernel library is not built.
    """
    import torch

    n = len(record)
    coded = DENSE_BYTES + HEADER_BYTES <= n <= DENSE_BYTES + VAR_CAP and n % 16 == 0
    if n != RAW_RECORD_BYTES and not coded:
        raise ValueError(f"{n} bytes is not a record length")
    if not torch.cuda.is_available():
        from fragpack_b200.compression import host_codec

        return host_codec.decode(bytes(record), table, int(kv))
    from fragpack_b200.ops.fragpack_ext import check, extension, stream_ptr

    dev = torch.device("cuda", torch.cuda.current_device())
    buf = torch.zeros(RAW_RECORD_BYTES, dtype=torch.uint8, device=dev)
    buf[:n] = torch.from_numpy(np.frombuffer(record, np.uint8).copy()).to(dev)
    plut, slut = _device_luts(table)
    which = torch.tensor([int(kv)], dtype=torch.int32, device=dev)
    length = torch.tensor([n - DENSE_BYTES], dtype=torch.int32, device=dev)
    out = torch.empty((PAGE_TOKENS, HEAD_DIM), dtype=torch.int16, device=dev)
    check(
        extension().fp_decode_records(
            buf.data_ptr(), RAW_RECORD_BYTES, length.data_ptr(), 1, plut.data_ptr(),
            slut.data_ptr(), None, which.data_ptr(), out.data_ptr(), stream_ptr(),
        )
    )
    return out.cpu().numpy().view(np.uint16)


def blob_head_bytes(num_layers: int, kv_heads: int) -> int:
    """Padded head (fixed header + length table) of a block blob (``attn_page.py:285-299``)."""
    head = BLOB_FIXED_BYTES + 8 * num_layers * kv_heads
    return -(-head // BLOB_ALIGN) * BLOB_ALIGN


def blob_slot_bytes(num_layers: int, kv_heads: int) -> int:
    """Largest block blob: every record raw (``attn_page.py:302-319``)."""
    return blob_head_bytes(num_layers, kv_heads) + 2 * num_layers * kv_heads * RAW_RECORD_BYTES


__all__ = [
    "BLOB_ALIGN",
    "BLOB_FIXED_BYTES",
    "BLOB_MAGIC",
    "DENSE_BYTES",
    "HEAD_DIM",
    "PAGE_TOKENS",
    "RAW_RECORD_BYTES",
    "VAR_CAP",
    "blob_head_bytes",
    "blob_slot_bytes",
    "calibrate_table",
    "decode_record",
    "encode_record",
    "primary_lut",
    "rank_table",
    "secondary_lut",
]
