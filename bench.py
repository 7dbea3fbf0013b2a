"""Headline benchmark: decode attention over HBM-resident compressed KV.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c3|c4|c5] [--arm fused|plain] [--layers R] [--no-graph]

A "step" is one decode step of the workload: the plan is computed once, then
every resident layer runs fused decode attention (one query token per
sequence).  With N = 1 the workload is the Qwen3-30B-A3B-like configuration
(48 layers, 4 KV heads, GQA 8, batch 4 at context 8192); with N > 1 it is the
Llama-3-70B-like configuration (8 KV heads, GQA 8, batch 128 at context 32768)
sharded by KV head, one process per GPU, with the per-head outputs all-gathered
over NCCL into the o_proj input layout after every layer.

Rank 0 prints ONE JSON line.  ``value`` is the effective logical-KV bandwidth
(BF16 bytes of the KV attended per second, whole job), measured with the KV
resident in HBM; ``e2e`` is the same metric through the public API with host
buffers (queries, lengths and block tables copied in, outputs copied out, per
step); ``roofline`` rates the decode kernel on COMPRESSED bytes against the
measured HBM copy bandwidth; ``cpu_baseline`` times the CPU oracle codec plus
torch CPU fp32 attention on a bounded sample of the same workload.

``--impl reference`` runs that CPU pipeline alone (all host threads) as the
reference arm.  ``--arm plain`` runs the comparison kernel: the same KV stored
as raw BF16 records and read by the same kernel template without the decode
step (what a plain BF16 paged read of the same logical KV costs).
``--impl reference-gpu`` runs the reference's own CUDA kernels (built unmodified
for sm_100a by oracle/build_ref_kernels.py) over the same records in the same
harness: the same-GPU kernel comparison.
``--workload c4`` measures the prefill side (token write, block encode,
decompression) instead.
"""

from __future__ import annotations

import argparse
import atexit
import datetime
import json
import os
from pathlib import Path
import subprocess
import sys
import time

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from fragpack_b200 import workloads  # noqa: E402
from fragpack_b200.compression import attn_page as ap  # noqa: E402

METRIC = "decode_attn_effective_logical_kv_bandwidth"
UNIT = "TB/s"
SCALE = 128**-0.5
L2_BYTES = 126 * 2**20
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_attn_kernel launch,
# from the ncu captures summarised under profiles/ (configuration 2 measured
# directly; the others are not captured at full size).
NCU_DRAM_BYTES_PER_LAUNCH = {"c2": 47_637_760 + 46_080 + 100_864}


def measured_hbm_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the GPU is under load.

    One ``nvidia-smi`` process in loop mode runs from :meth:`start` (early: it
    needs a moment before its first sample) to :meth:`stop`; :meth:`mark_begin`
    and :meth:`mark_end` bracket the loaded region, and only the samples whose
    own timestamps fall inside it are summarised.
    """

    FIELDS = (
        "timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int, period_ms: int = 25) -> None:
        self.index = index
        self.period_ms = period_ms
        self.rows: list[list[str]] = []
        self._proc: subprocess.Popen | None = None
        self._begin = self._end = None

    def start(self) -> "ClockSampler":
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self._proc = None
        atexit.register(self.stop)  # the child must not outlive a failed run
        return self

    def mark_begin(self) -> None:
        self._begin = datetime.datetime.now()

    def mark_end(self) -> None:
        self._end = datetime.datetime.now()

    def stop(self) -> None:
        if self._proc is None:
            return
        self._proc.terminate()
        try:
            out, _ = self._proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            self._proc.kill()
            out, _ = self._proc.communicate()
        self._proc = None
        self.rows = [[c.strip() for c in line.split(",")] for line in out.splitlines() if line.strip()]

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in self.rows:
            try:
                when = datetime.datetime.strptime(row[0], "%Y/%m/%d %H:%M:%S.%f")
                if self._begin and self._end and not (self._begin <= when <= self._end):
                    continue
                sm.append(float(row[1]))
                mx.append(float(row[2]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, row[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": float(np.median(sm)) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
            "window": "warm-up, timed steps, per-launch timing and end-to-end steps",
        }


# --------------------------------------------------------------------------
# CPU pipeline (oracle codec + torch fp32 attention): baseline and reference arm
# --------------------------------------------------------------------------
def cpu_pipeline(sample: dict, repeats: int = 1) -> tuple[float, float, int]:
    """Decode the sample's records on the host cores and attend over them.

    Args:
        sample: ``records u8[n,32768]``, ``lens i32[n]``, ``tables u8[n,22]``,
            ``kv i32[n]``, ``q`` float32 ``[n_seq_heads, G, 128]``, ``pages``
            per (sequence, head) record ranges, ``seq_lens``.

    Returns:
        ``(seconds, logical_bytes, threads)`` for one pass.
    """
    import oracle

    t0 = time.perf_counter()
    for _ in range(repeats):
        dec = oracle.decode_records(sample["records"], sample["lens"], sample["tables"], sample["kv"])
        f32 = torch.from_numpy(oracle.bf16_bits_to_f32(dec))  # [n,128,128]
        for (k0, k1, v0, v1, tokens), q in zip(sample["ranges"], sample["q"]):
            k = f32[k0:k1].reshape(-1, 128)[:tokens]
            v = f32[v0:v1].reshape(-1, 128)[:tokens]
            oracle.attention_fp32(q, k, v, SCALE)
    seconds = (time.perf_counter() - t0) / repeats
    return seconds, float(sample["logical_bytes"]), oracle.threads()


def sample_for_cpu(work: workloads.DecodeWorkload, layers: int, seqs: int) -> dict:
    """Copy the records of ``layers`` x ``seqs`` sequences to the host (all heads)."""
    store, cfg = work.store, work.cfg
    heads = cfg.kv_heads
    records, lens, tables, kvs, ranges, qs = [], [], [], [], [], []
    bt = work.block_table.cpu().numpy()
    rec_addr = store.rec_addr.cpu().numpy()
    rec_len = store.rec_len.cpu().numpy()
    gen = torch.Generator().manual_seed(7)
    logical = 0
    at = 0

    pools = [(t.data_ptr(), t.numel(), t.view(-1)) for t in
             (*work.arenas, store.staging, store.scratch, store.overflow, store.null_record)]

    def fetch(addr: int, n: int) -> np.ndarray:
        # A record lives in an arena page, in staging, in the overflow pool or
        # is the shared null record: find the pool that holds its address.
        for base, size, flat in pools:
            if base <= addr < base + size:
                out = np.zeros(32768, np.uint8)
                out[:n] = flat[addr - base : addr - base + n].cpu().numpy()
                return out
        raise RuntimeError("record address outside every pool")

    for layer in range(layers):
        for b in range(seqs):
            tokens = int(work.lens_host[b])
            pages = (tokens + 127) // 128
            for h in range(heads):
                span = []
                for kv in range(2):
                    first = at
                    for pg in range(pages):
                        blk = bt[b, pg]
                        n = int(rec_len[layer, blk, kv, h]) + ap.DENSE_BYTES
                        records.append(fetch(int(rec_addr[layer, blk, kv, h]), n))
                        lens.append(n)
                        tables.append(work.table[layer, kv, h])
                        kvs.append(kv)
                        at += 1
                    span += [first, at]
                ranges.append((span[0], span[1], span[2], span[3], tokens))
                qs.append(torch.randn(cfg.group, 128, generator=gen))
                logical += tokens * 2 * 128 * 2
    return {
        "records": np.stack(records),
        "lens": np.array(lens, np.int32),
        "tables": np.stack(tables),
        "kv": np.array(kvs, np.int32),
        "ranges": ranges,
        "q": qs,
        "logical_bytes": logical,
        "what": f"{layers} layer(s) x {seqs} sequence(s) x {heads} KV heads of {cfg.name}",
    }


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def validate(work, queries, outputs, layer: int) -> tuple[float, float]:
    """Max / mean abs error of ``outputs[layer]`` vs fp32 attention over the kept source KV."""
    cfg = work.cfg
    worst, total, count = 0.0, 0.0, 0
    for (lay, b), kv in work.sample.items():
        if lay != layer:
            continue
        k = kv[0].float()  # [T, H, 128]
        v = kv[1].float()
        for h in range(cfg.kv_heads):
            q = queries[layer][b, h * cfg.group : (h + 1) * cfg.group].float()
            ref = torch.softmax(q @ k[:, h].T * SCALE, -1) @ v[:, h]
            err = (outputs[layer][b, h * cfg.group : (h + 1) * cfg.group].float() - ref).abs()
            # The bar is absolute for outputs up to magnitude 1 and relative above
            # it: BF16 outputs near 100 (x64 heavy-tail V) are spaced 0.5 apart.
            err = err / ref.abs().clamp(min=1.0)
            worst = max(worst, float(err.max()))
            total += float(err.sum())
            count += err.numel()
    return worst, total / max(count, 1)


def run_ours(args) -> dict:
    from fragpack_b200.ops.fused_attn_decode import (
        RecordTables,
        decode_attention,
        decode_status,
        decode_units,
        plain_decode_attention,
        workspace_elems,
    )

    plain = args.arm == "plain"
    refgpu = args.impl == "reference-gpu"
    if plain:
        # Comparison arm: every record raw BF16, read by the kernel without a
        # decode step.  Same planner, pipeline, softmax, merge and harness.
        decode_attention = plain_decode_attention
    if refgpu:
        # Comparison arm: the reference's own kernels (built unmodified for
        # sm_100a into oracle/_ref) reading the records this library wrote.
        from oracle import build_ref_kernels

        try:
            ref_mod = build_ref_kernels.module()
        except Exception as exc:  # noqa: BLE001
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference-gpu",
                                  "unavailable": f"the reference's CUDA extension is not built here: {exc}"}))
            raise SystemExit(0)

        def decode_attention(q, tabs, block_table, seq_lens, scale, units, out, ws, replan):
            # The reference's host wrapper (fragpack/ops/fused_attn_decode.py:105-171):
            # its kernel attends 8 query heads per KV head; smaller groups run
            # zero-padded and are copied back.
            kvh = tabs.rec_addr.shape[2]
            group = q.shape[1] // kvh
            if group == 8:
                ref_mod.fused_decode(q, tabs.rec_addr, tabs.rec_len, tabs.plut, tabs.slut, block_table,
                                     seq_lens, ws[0], ws[1], ws[2], out, units, replan, scale)
                return
            qp = q.new_zeros(q.shape[0], kvh, 8, 128)
            qp[:, :, :group] = q.unflatten(1, (kvh, group))
            op = torch.empty_like(qp)
            ref_mod.fused_decode(qp.flatten(1, 2), tabs.rec_addr, tabs.rec_len, tabs.plut, tabs.slut,
                                 block_table, seq_lens, ws[0], ws[1], ws[2], op.flatten(1, 2), units,
                                 replan, scale)
            out.unflatten(1, (kvh, group)).copy_(op[:, :, :group])

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    clocks = ClockSampler(local).start()
    name = args.workload or ("c2" if world == 1 else "c5")
    cfg = workloads.CONFIGS[name]
    if args.batch or args.ctx:
        # Reduced copies of a configuration, for profiler captures.
        from dataclasses import replace

        ctx = args.ctx or cfg.ctx_max
        cfg = replace(cfg, name=f"{cfg.name}-reduced", batch=args.batch or cfg.batch,
                      ctx_min=min(cfg.ctx_min, ctx), ctx_max=ctx)
    if cfg.kv_heads % world:
        raise SystemExit(f"{world} GPUs do not divide {cfg.kv_heads} KV heads")
    per = cfg.kv_heads // world
    head_slice = slice(rank * per, (rank + 1) * per)
    # Resident layers: all of them when they fit, else as many as the budget holds.
    per_layer = cfg.batch * ((cfg.ctx_max + 127) // 128) * 2 * per * (ap.DENSE_BYTES + 1280)
    if plain:
        per_layer += cfg.batch * ((cfg.ctx_max + 127) // 128) * 2 * per * ap.RAW_RECORD_BYTES
    budget = int(args.hbm_budget_gb * 2**30)
    layers = args.layers or max(1, min(cfg.layers, budget // max(per_layer, 1)))
    if world > 1 and layers > 2:
        # An even count keeps the two gathered copies alternating inside a replayed graph.
        layers -= layers % 2
    work = workloads.build_decode_workload(
        cfg, device, seed=args.seed, layers=layers, head_slice=head_slice,
        keep_layers=(0, layers - 1), plain=plain,
    )
    cfg_built = work.cfg
    B, H, G = cfg_built.batch, cfg_built.kv_heads, cfg_built.group
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = decode_units(B, H, sms)
    if refgpu:
        # The reference reserves one wave of split capacity (fused_attn_decode.py:58-85).
        units = B + max(1, (2 * sms) // H) - 1
    sizes = workspace_elems(H, units)
    ws = (
        torch.empty(sizes[0], device=device),
        torch.empty(sizes[1], device=device),
        torch.empty(sizes[2], dtype=torch.int32, device=device),
    )
    gen = torch.Generator(device=device).manual_seed(args.seed + 100 + rank)
    # One tensor for all layers' queries and one for their outputs, so that the
    # end-to-end step moves each with a single copy; a layer's call sees its slice.
    q_all = torch.randn(layers, B, H * G, 128, generator=gen, device=device).to(torch.bfloat16)
    out_all = torch.full_like(q_all, float("nan"))
    queries = [q_all[layer] for layer in range(layers)]
    outputs = [out_all[layer] for layer in range(layers)]
    tabs = [RecordTables(*work.store.layer_tables(layer)) for layer in range(layers)]
    gather = peer_gather = None
    if world > 1 and not plain and not refgpu and args.gather == "peers":
        from fragpack_b200.ops.tp import PeerGather

        # The merge kernel stores this rank's heads into every rank's o_proj
        # input over NVLink (peer pointers) and waits for the other ranks.
        # Mapping peer memory can be refused by a container; every rank then
        # uses the collective instead (the line's `parallelism` says which ran).
        try:
            peer_gather = PeerGather(B, H * G, device)
            mapped = 1
        except Exception as exc:  # noqa: BLE001
            print(f"[rank {rank}] peer mapping failed ({exc}); using the NCCL all-gather", file=sys.stderr)
            mapped = 0
        agreed = torch.tensor([mapped], device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if not int(agreed.item()):
            peer_gather = None
    if world > 1 and peer_gather is None:
        from fragpack_b200.ops.tp import HeadGather

        gather = HeadGather(B, H * G, torch.bfloat16, device)
    oproj_in = None

    def attend(layer: int) -> None:
        decode_attention(queries[layer], tabs[layer], work.block_table, work.seq_lens, SCALE,
                         units, outputs[layer], ws, replan=layer == 0)

    def step() -> None:
        nonlocal oproj_in
        for layer in range(layers):
            if peer_gather is not None:
                oproj_in = peer_gather.decode(queries[layer], tabs[layer], work.block_table,
                                              work.seq_lens, SCALE, units, ws, replan=layer == 0)
                continue
            attend(layer)
            if gather is not None:
                # Per-head outputs -> o_proj input layout [B, Hq, 128] on every rank.
                oproj_in = gather(outputs[layer])

    # Correctness gate before any timing (outputs start as NaN).
    step()
    torch.cuda.synchronize()
    if not refgpu and decode_status(ws, units):
        raise SystemExit("decode kernel reported a timed-out wait")
    if peer_gather is not None:
        if peer_gather.status():
            raise SystemExit("a peer did not arrive within the wait limit")
        # The gathered copy of the last layer holds this rank's heads where the
        # validation below expects them.
        lo = rank * H * G
        last = (layers - 1) & 1
        outputs[layers - 1].copy_(peer_gather.gathered[last][:, lo : lo + H * G])
        if layers > 1:
            # Layer 0's copy has been overwritten by later layers; recompute it locally.
            attend(0)
        torch.cuda.synchronize()
    worst = mean = 0.0
    for layer in (0, layers - 1):
        w, m = validate(work, queries, outputs, layer)
        worst, mean = max(worst, w), max(mean, m)
    # With the peer-store gather the layers' results live in the two gathered
    # copies; only the validated layers were copied back into `outputs`.
    checked = outputs if peer_gather is None else [outputs[0], outputs[layers - 1]]
    failed = not (worst <= 1e-2 and mean <= 2e-3) or any(torch.isnan(o).any() for o in checked)
    if failed and not args.skip_validation:
        raise SystemExit(f"validation failed: max-abs {worst:.3e}, mean-abs {mean:.3e}")

    # NCCL calls stay out of the graph; the peer-store gather is plain kernels
    # (an even number of calls per replay keeps its two copies alternating).
    use_graph = not args.no_graph and (world == 1 or (peer_gather is not None and layers % 2 == 0))
    graph = None
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()

    def run_step() -> None:
        if graph is not None:
            graph.replay()
        else:
            step()

    def barrier() -> None:
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    clocks.mark_begin()
    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        run_step()
    stop.record()
    barrier()
    ms = start.elapsed_time(stop)
    if dist is not None:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps

    # Per-launch duration of the decode call of every layer, events on the
    # launching stream (no graph), for the roofline of the dominant kernel.
    per_call = []
    for _ in range(3):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(layers + 1)]
        decode_attention(queries[0], tabs[0], work.block_table, work.seq_lens, SCALE, units,
                         outputs[0], ws, replan=True)
        evs[0].record()
        for layer in range(layers):
            decode_attention(queries[layer], tabs[layer], work.block_table, work.seq_lens, SCALE,
                             units, outputs[layer], ws, replan=False)
            evs[layer + 1].record()
        torch.cuda.synchronize()
        per_call.append(np.mean([evs[i].elapsed_time(evs[i + 1]) for i in range(layers)]))
    call_ms = float(np.min(per_call))
    if use_graph:
        # Eager calls are paced by the host (one ctypes call per layer), so their
        # event spacing includes host gaps.  Inside the replayed graph a layer is
        # exactly the attention kernel followed by the small merge kernel: use
        # that time (an upper bound on the attention kernel's own duration).
        call_ms = min(call_ms, ms_per_step / layers)

    # End to end through the public API with host buffers.
    q_host = q_all.cpu().pin_memory()
    out_host = torch.empty_like(q_all, device="cpu").pin_memory()
    bt_host = work.block_table.cpu().pin_memory()
    len_host = work.seq_lens.cpu().pin_memory()
    h2d = q_host.numel() * 2 + bt_host.numel() * 4 + len_host.numel() * 4
    d2h = out_host.numel() * 2

    def e2e_step() -> None:
        work.block_table.copy_(bt_host, non_blocking=True)
        work.seq_lens.copy_(len_host, non_blocking=True)
        q_all.copy_(q_host, non_blocking=True)
        run_step()
        if peer_gather is not None:
            # The result lives in the two gathered copies (the last two layers');
            # read this rank's heads of each back, the same bytes per layer.
            lo = rank * H * G
            for layer in range(layers):
                out_host[layer].copy_(peer_gather.gathered[layer & 1][:, lo : lo + H * G], non_blocking=True)
        else:
            out_host.copy_(out_all, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if dist is not None:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    clocks.mark_end()
    clocks.stop()

    logical_all = work.logical_bytes * layers * world  # every rank holds an equal head shard
    compressed_layer = float(np.mean(work.compressed_bytes))
    peak, peak_kind = measured_hbm_peak()
    achieved = compressed_layer / (call_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC,
        "value": logical_all / (ms_per_step * 1e-3) / 1e12,
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None,
        "dtype": "bf16 KV and P, fp32 softmax/accumulate; u8/u32 integer decode",
        "data": "synthetic (seeded per-channel lognormal-scaled Gaussian BF16 KV, K outlier channels)",
        "config": {
            "workload": cfg.name,
            "arm": ("the reference's CUDA kernels built for sm_100a, reading this library's records (comparison)"
                    if refgpu else "plain BF16 records, no decode step (comparison)" if plain
                    else "fused decode over compressed records"),
            "layers_resident": layers,
            "layers_model": cfg.layers,
            "kv_heads_per_gpu": H,
            "q_heads_per_gpu": H * G,
            "batch": B,
            "context": [int(work.lens_host.min()), int(work.lens_host.max())],
            "parallelism": f"kv-head shard tp{world}" + (
                "" if world == 1 else
                " + output gather by the merge kernel (peer stores over NVLink)" if peer_gather is not None
                else " + NCCL all-gather per layer"),
            "cuda_graph": bool(use_graph),
            "l2_policy": "inputs larger than L2: every layer reads distinct pages, "
                         f"{compressed_layer * layers / 2**20:.0f} MiB per step vs 126 MiB L2",
        },
        "us_per_layer": ms_per_step * 1e3 / layers,
        "kv_ratio": work.logical_bytes / compressed_layer,
        "compressed_gbs": compressed_layer * layers * world / (ms_per_step * 1e-3) / 1e9,
        "e2e": {
            "value": logical_all / (e2e_ms * 1e-3) / 1e12,
            "unit": UNIT,
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "ms_per_step": e2e_ms,
        },
        # This library's kernels per step: one planner, then attention + merge per layer.
        "gpu_launches": 0 if refgpu else args.steps * (1 + (4 if peer_gather is not None else 2) * layers),
        "roofline": {
            "bound": "hbm",
            "kernel": ("reference decode_attn" if refgpu else "plain_attn_kernel" if plain
                       else "decode_attn_kernel") + " (duration includes the merge kernel that follows it)",
            "achieved": achieved,
            "peak": peak,
            "peak_kind": peak_kind,
            "unit": "GB/s",
            "frac": achieved / peak,
            "traffic": (NCU_DRAM_BYTES_PER_LAUNCH.get(name)
                        if not (args.batch or args.ctx or plain or refgpu) else None),
            "algorithmic_bytes_per_launch": compressed_layer,
            "launch_ms": call_ms,
        },
        "validation": {"max_abs": worst, "mean_abs": mean},
        "clocks": clocks.summary(),
    }
    if refgpu:
        line["impl"] = "reference-gpu"
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not plain and not refgpu:
        sample = sample_for_cpu(work, layers=min(layers, args.cpu_layers), seqs=min(B, args.cpu_seqs))
        first, logical, threads = cpu_pipeline(sample)
        passes = max(1, int(np.ceil(args.cpu_seconds / max(first, 1e-3))))
        seconds, logical, threads = cpu_pipeline(sample, repeats=passes)
        line["cpu_baseline"] = {
            "value": logical / seconds / 1e12,
            "unit": UNIT,
            "cores": threads,
            "kind": "port",
            "sample": sample["what"] + f" ({len(sample['lens'])} records; {passes} timed passes of "
                      f"{seconds:.2f} s each after one warm-up pass)",
        }
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else {}


def run_codec(args) -> dict:
    """Prefill side (configuration 4): token write + block encode, then decompression.

    One step = one layer of the MHA stress geometry (32 KV heads, 16 x 8192
    tokens = 1024 blocks): the tokens are scattered into staging, every completed
    block is encoded into its arena page, and all blocks are decompressed into the
    BF16 workspace.  Each phase is timed with CUDA events on its own.
    """
    from fragpack_b200 import synth
    from fragpack_b200.compression.attn_tables import device_tables
    from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    cfg = workloads.CONFIGS["c4"]
    junk = args.junk if args.junk >= 0 else 0.009
    heads, layers = cfg.kv_heads, args.layers or 2
    tokens = (args.batch or cfg.batch) * (args.ctx or cfg.ctx_max)
    blocks = tokens // 128
    scales = synth.channel_scales(args.seed + 1, layers, heads)
    gen = torch.Generator(device=device).manual_seed(args.seed + 4)
    scales_dev = torch.from_numpy(scales).to(device)
    table = np.stack([workloads.calibrate_on_device(gen, scales_dev[layer], 0.0, junk)
                      for layer in range(layers)])
    arenas = [torch.empty((blocks + 1, page_bytes(heads)), dtype=torch.uint8, device=device)
              for _ in range(layers)]
    store = HbmKvStore(arenas, heads, device_tables(table, device), max_tokens=tokens,
                       staging_slots=1, overflow_records=args.overflow)
    ids = torch.from_numpy(np.random.default_rng(args.seed).permutation(np.arange(1, blocks + 1)))
    slots = (ids.repeat_interleave(128) * 128 + torch.arange(128).repeat(blocks)).to(device)
    ids_dev = ids.to(torch.int32).to(device)
    wk = torch.empty(blocks, 128, heads, 128, dtype=torch.bfloat16, device=device)
    wv = torch.empty_like(wk)
    kv = [synth.kv_tokens_torch(gen, scales_dev[layer], tokens, 0.0, junk) for layer in range(layers)]
    times = {"write": [], "encode": [], "gather": []}
    ok = True
    for it in range(max(args.warmup, 1) + args.steps):
        store.prepare(slots, tokens, np.zeros(0, np.int32))
        for layer in range(layers):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
            store.write(layer, kv[layer][0], kv[layer][1], slots)
            ev[1].record()
            store.encode(layer, blocks)
            ev[2].record()
            store.gather(layer, ids_dev, wk, wv)
            ev[3].record()
            torch.cuda.synchronize()
            if it >= max(args.warmup, 1):
                for name, a, b in (("write", 0, 1), ("encode", 1, 2), ("gather", 2, 3)):
                    times[name].append(ev[a].elapsed_time(ev[b]))
            if it == 0:
                # Bit-exact reconstruction of what was written.
                src_k = kv[layer][0].view(blocks, 128, heads, 128)
                src_v = kv[layer][1].view(blocks, 128, heads, 128)
                ok &= bool(torch.equal(wk, src_k)) and bool(torch.equal(wv, src_v))
        store.commit()
    counters = store.counters.cpu().numpy()
    records = blocks * 2 * heads
    rec_bytes = float((store.rec_len[0, ids_dev.long()].to(torch.int64) + ap.DENSE_BYTES).sum().item())
    peak, peak_kind = measured_hbm_peak()
    ms = {k: float(np.mean(v)) for k, v in times.items()}
    enc_bytes = records * 32768 + rec_bytes
    dec_bytes = rec_bytes + records * 32768
    return {
        "metric": "block_encode_and_decompress_throughput",
        "value": enc_bytes / (ms["encode"] * 1e-3) / 1e9,
        "unit": "GB/s (encode: raw bytes read + record bytes written)",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": max(args.warmup, 1),
        "ms_per_step": ms["write"] + ms["encode"] + ms["gather"],
        "higher_is_better": True,
        "config": {"workload": cfg.name, "layers_resident": layers, "kv_heads": heads,
                   "tokens_per_layer": tokens, "blocks_per_layer": blocks, "junk_fraction": junk,
                   "overflow_records": args.overflow},
        "bit_exact_roundtrip": ok,
        "mean_record_bytes": rec_bytes / records,
        "counters": {"encoded": int(counters[7]), "fallbacks": int(counters[6]),
                     "spills": int(counters[8]), "err_overflow": int(counters[5]),
                     "err_staging": int(counters[4])},
        "write": {"ms_per_layer": ms["write"],
                  "GBps": (records * 32768 * 2) / (ms["write"] * 1e-3) / 1e9},
        "encode": {"ms_per_layer": ms["encode"], "GBps": enc_bytes / (ms["encode"] * 1e-3) / 1e9,
                   "roofline_frac": enc_bytes / (ms["encode"] * 1e-3) / 1e9 / peak},
        "decompress": {"ms_per_layer": ms["gather"], "GBps": dec_bytes / (ms["gather"] * 1e-3) / 1e9,
                       "roofline_frac": dec_bytes / (ms["gather"] * 1e-3) / 1e9 / peak},
        "peak": peak, "peak_kind": peak_kind,
    }


def run_reference(args) -> dict:
    """Reference arm: the CPU codec (oracle port) + torch CPU fp32 attention."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return {}
    import oracle
    from fragpack_b200 import synth

    name = args.workload or ("c2" if world == 1 else "c5")
    cfg = workloads.CONFIGS[name]
    # Bounded sample of the workload: one layer, a few (sequence, head) pairs.
    rng = np.random.default_rng(args.seed)
    scales = synth.channel_scales(args.seed + 1, 1, cfg.kv_heads)[0]
    tokens = min(cfg.ctx_max, 8192)
    pairs = args.cpu_pairs
    dump = synth.calibration_dump(args.seed + 4, scales[None], 16)
    table = oracle.calibrate(dump)[0]
    records, tables, kvs, ranges, qs = [], [], [], [], []
    at = 0
    pages = tokens // 128
    for pair in range(pairs):
        h = pair % cfg.kv_heads
        kv = synth.kv_tokens_numpy(rng, scales[:, h : h + 1], tokens, cfg.heavy, cfg.junk)
        span = []
        for k in range(2):
            first = at
            for pg in range(pages):
                records.append(kv[k, pg * 128 : (pg + 1) * 128, 0])
                tables.append(table[k, h])
                kvs.append(k)
                at += 1
            span += [first, at]
        ranges.append((span[0], span[1], span[2], span[3], tokens))
        qs.append(torch.randn(cfg.group, 128))
    enc, lens = oracle.encode_records(np.stack(records), np.stack(tables), np.array(kvs, np.int32))
    sample = {
        "records": enc, "lens": lens, "tables": np.stack(tables), "kv": np.array(kvs, np.int32),
        "ranges": ranges, "q": qs, "logical_bytes": pairs * tokens * 2 * 128 * 2,
    }
    for _ in range(max(args.warmup, 1)):
        cpu_pipeline(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        seconds, logical, threads = cpu_pipeline(sample)
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    value = logical / (ms * 1e-3) / 1e12
    what = f"{pairs} (sequence, KV head) pairs x {tokens} tokens of one layer of {cfg.name} per step"
    return {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 1),
        "ms_per_step": ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "u8/u16 integer decode, fp32 attention",
        "data": "synthetic",
        "config": {"workload": cfg.name, "sample": what},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference", "reference-gpu"), default="ours",
                        help="reference: the CPU codec + attention (the reference arm); reference-gpu: the "
                             "reference's own CUDA kernels built for sm_100a (extra comparison, 1 GPU)")
    parser.add_argument("--workload", choices=("c2", "c3", "c4", "c5"), default=None)
    parser.add_argument("--arm", choices=("fused", "plain"), default="fused",
                        help="plain: the comparison kernel over raw BF16 records of the same KV")
    parser.add_argument("--junk", type=float, default=-1.0, help="c4: junk fraction (default 0.009)")
    parser.add_argument("--overflow", type=int, default=8192, help="c4: overflow records")
    parser.add_argument("--gather", choices=("peers", "nccl"), default="peers",
                        help="N > 1: how the per-rank outputs reach every rank's o_proj input")
    parser.add_argument("--layers", type=int, default=0, help="resident layers (default: what fits)")
    parser.add_argument("--hbm-budget-gb", type=float, default=40.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--batch", type=int, default=0, help="override the batch (profiling)")
    parser.add_argument("--ctx", type=int, default=0, help="override the context (profiling)")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--skip-validation", action="store_true",
                        help="keep going when the correctness gate fails (kernel experiments only)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--cpu-layers", type=int, default=8)
    parser.add_argument("--cpu-seqs", type=int, default=4)
    parser.add_argument("--cpu-pairs", type=int, default=64,
                        help="reference arm: (sequence, KV head) pairs decoded and attended per step")
    parser.add_argument("--cpu-seconds", type=float, default=12.0,
                        help="CPU baseline: seconds of host work to time")
    args = parser.parse_args()
    if args.workload == "c4" and args.impl == "ours":
        line = run_codec(args)
    else:
        line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
