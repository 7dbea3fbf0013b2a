"""Host (numpy) form of the FragPack record codec.

The serving path never uses this module: ``fragpack_b200.ops`` has no CPU
fallback.  It exists so that ``fragpack_b200.compression`` works where the
reference's ``fragpack.compression`` does - offline tools, calibration
machines and unit tests without a CUDA device.  It produces and consumes
exactly the bytes of the reference codec (``fragpack/compression/attn_page.py``
``encode_record`` :146-209, ``decode_record`` :212-269) and of the sm_100a
kernels, and is written from the record format, array-at-a-time.

Fragment order: position ``p = 64 t + s`` belongs to owner ``t`` (warp
``w = t >> 5``, ``g = (t >> 2) & 7``, ``c = t & 3``) with
``s = 8 st + 4 j + 2 f + e``; for K it holds token ``16 w + 8 j + g``, dim
``16 st + 8 f + 2 c + e``; for V token ``16 st + 8 f + 2 c + e``, dim
``16 w + 8 j + g``.
"""

from __future__ import annotations

import functools

import numpy as np
from numpy.typing import NDArray

OWNERS = 256
SCALARS = 16384
LOW_BYTES = 16384
SYMBOL_BYTES = 6144
DENSE_BYTES = LOW_BYTES + SYMBOL_BYTES
HEADER_BYTES = 48
VAR_CAP = 2048
RAW_BYTES = 32768
DIRECT = 7
MAX_WARP_RAW = 32


@functools.cache
def fragment_order(kv: int) -> NDArray[np.int64]:
    """Token-major index ``128 * token + dim`` of every fragment-order position."""
    p = np.arange(SCALARS)
    t, s = p >> 6, p & 63
    w, g, c = t >> 5, (t >> 2) & 7, t & 3
    st, j, f, e = s >> 3, (s >> 2) & 1, (s >> 1) & 1, s & 1
    row = 16 * w + 8 * j + g
    col = 16 * st + 8 * f + 2 * c + e
    token, dim = (row, col) if kv == 0 else (col, row)
    return (128 * token + dim).astype(np.int64)


def _raw_bytes(frag: NDArray[np.uint16]) -> bytes:
    """Fragment-order scalars as a raw record: word ``st`` of owner ``t`` at ``16 (256 st + t)``."""
    return np.ascontiguousarray(frag.reshape(OWNERS, 8, 8).transpose(1, 0, 2)).astype("<u2").tobytes()


def encode(raw: NDArray[np.uint16], rank_of: NDArray[np.uint8], kv: int) -> bytes:
    """Encode one token-major ``[128, 128]`` record; returns the record bytes."""
    frag = np.ascontiguousarray(raw, dtype=np.uint16).reshape(-1)[fragment_order(kv)]
    high = (frag >> 8).astype(np.uint8)
    low = (frag & 0xFF).astype(np.uint8)
    rank = rank_of[high].astype(np.int64)
    code = np.minimum(rank, DIRECT)

    # Escapes in fragment order: one nibble each, raw ones also on the raw list.
    escaped = np.flatnonzero(code == DIRECT)
    nibble = np.where(rank[escaped] == 255, 15, rank[escaped] - DIRECT)
    is_raw = nibble == 15
    n_esc, n_raw = int(escaped.size), int(is_raw.sum())
    raw_offset = (HEADER_BYTES + (n_esc + 1) // 2 + 3) & ~3
    var_len = (raw_offset + 4 * n_raw + 15) & ~15
    warp_of = escaped >> 11
    esc_per_warp = np.bincount(warp_of, minlength=8)
    raw_per_warp = np.bincount(warp_of[is_raw], minlength=8)
    if var_len > VAR_CAP or raw_per_warp.max(initial=0) > MAX_WARP_RAW:
        return _raw_bytes(frag)

    out = np.zeros(DENSE_BYTES + var_len, np.uint8)
    # Low bytes: 16-byte chunk j of owner t at 16 (256 j + t).
    out[:LOW_BYTES] = low.reshape(OWNERS, 4, 16).transpose(1, 0, 2).reshape(-1)
    # Codes: per owner and 32-scalar group three words; nibble n of word k is the
    # code of scalar 8 k + n, with bit k of the code of scalar 24 + n on top.
    groups = code.reshape(OWNERS, 2, 4, 8)
    nibbles = groups[:, :, :3, :] | (((groups[:, :, 3:4, :] >> np.arange(3)[None, None, :, None]) & 1) << 3)
    words = (nibbles.astype(np.uint32) << (4 * np.arange(8, dtype=np.uint32))).sum(-1, dtype=np.uint32)
    # An owner's six words as three 8-byte chunks, chunk m at 16384 + 8 (256 m + t).
    chunks = words.reshape(OWNERS, 3, 2).transpose(1, 0, 2)
    out[LOW_BYTES:DENSE_BYTES] = np.ascontiguousarray(chunks).astype("<u4").view(np.uint8).reshape(-1)

    var = out[DENSE_BYTES:]
    header = np.zeros(4, "<u4")
    header[:3] = (n_esc, n_raw, raw_offset)
    var[:16] = header.view(np.uint8)
    prefixes = np.zeros(16, "<u2")
    prefixes[:8] = np.cumsum(esc_per_warp) - esc_per_warp
    prefixes[8:] = np.cumsum(raw_per_warp) - raw_per_warp
    var[16:HEADER_BYTES] = prefixes.view(np.uint8)
    packed = np.zeros((n_esc + 1) // 2 * 2, np.uint8)
    packed[:n_esc] = nibble
    var[HEADER_BYTES : HEADER_BYTES + packed.size // 2] = packed[0::2] | (packed[1::2] << 4)
    entries = (np.flatnonzero(is_raw).astype(np.uint32) | (high[escaped[is_raw]].astype(np.uint32) << 16))
    var[raw_offset : raw_offset + 4 * n_raw] = entries.astype("<u4").view(np.uint8)
    return out.tobytes()


def decode(record: bytes, table: NDArray[np.uint8], kv: int) -> NDArray[np.uint16]:
    """Decode one record to token-major ``uint16 [128, 128]``.

    Raises:
        ValueError: If the record's variable region contradicts its codes.
    """
    buf = np.frombuffer(record, np.uint8)
    if buf.size == RAW_BYTES:
        frag = buf.view("<u2").reshape(8, OWNERS, 8).transpose(1, 0, 2).reshape(-1)
    else:
        low = buf[:LOW_BYTES].reshape(4, OWNERS, 16).transpose(1, 0, 2).reshape(-1)
        words = buf[LOW_BYTES:DENSE_BYTES].view("<u4").reshape(3, OWNERS, 2).transpose(1, 0, 2).reshape(OWNERS, 2, 3)
        nibbles = (words[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & 15
        fourth = ((nibbles >> 3) << np.arange(3, dtype=np.uint32)[None, None, :, None]).sum(2)
        code = np.concatenate([nibbles & 7, fourth[:, :, None, :]], axis=2).reshape(-1).astype(np.int64)
        var = buf[DENSE_BYTES:]
        n_esc, n_raw, raw_offset = (int(x) for x in var[:12].view("<u4"))
        escaped = np.flatnonzero(code == DIRECT)
        if escaped.size != n_esc or raw_offset + 4 * n_raw > var.size:
            raise ValueError("malformed record")
        packed = var[HEADER_BYTES : HEADER_BYTES + (n_esc + 1) // 2]
        nibble = np.stack([packed & 15, packed >> 4], -1).reshape(-1)[:n_esc].astype(np.int64)
        extended = np.zeros(16, np.uint8)
        extended[:15] = np.asarray(table, np.uint8)[DIRECT:]
        primary = np.zeros(8, np.uint8)
        primary[:DIRECT] = np.asarray(table, np.uint8)[:DIRECT]
        high = primary[code]
        high[escaped] = extended[nibble]
        entries = var[raw_offset : raw_offset + 4 * n_raw].view("<u4")
        if n_raw:
            ordinal = (entries & 0xFFFF).astype(np.int64)
            if ordinal.max() >= n_esc:
                raise ValueError("malformed record")
            high[escaped[ordinal]] = (entries >> 16).astype(np.uint8)
        frag = (high.astype(np.uint16) << 8) | low
    out = np.empty(SCALARS, np.uint16)
    out[fragment_order(kv)] = frag
    return out.reshape(128, 128)
