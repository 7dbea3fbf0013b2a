"""Headline benchmark: decode attention over HBM-resident compressed KV.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu]
                    [--workload c2|c3|c4|c5] [--arms fused,reference,plain] [--layers R] ...

A "step" is one decode step: the plan is computed once, then every resident
layer runs fused decode attention (one query token per sequence).  At every N
the workload is the Llama-3-70B-like configuration the metric is quoted on
(8 KV heads, GQA 8, batch 128 at context 32768), sharded by KV head over the N
GPUs, one process per GPU; as many of its 80 layers are resident as the HBM
budget holds (every layer reads distinct pages, so a step reads far more than
the L2).  With N > 1 the merge kernel writes each rank's heads into every
rank's o_proj input over NVLink (peer stores) after every layer.

Rank 0 prints ONE JSON line.  ``value`` is the effective logical-KV bandwidth
(BF16 bytes of the KV attended per second, whole job), measured with the KV
resident in HBM over exactly K steps; ``e2e`` is the same metric through the
public API with host buffers (queries, lengths and block tables copied in,
outputs copied out, per step); ``roofline`` rates the decode kernel on
COMPRESSED bytes against the measured HBM copy bandwidth; ``cpu_baseline``
times the CPU oracle codec plus torch CPU fp32 attention on a bounded sample
of the same workload.  ``arms`` compares, in this same process and with
interleaved rounds, the fused kernel with the reference's own CUDA kernels
(built unmodified for sm_100a, reading the same records) and with a plain
BF16 read of the same logical KV.  With N = 1 the line also carries ``extra``:
the same measurements on configurations 2 and 3 and the prefill side
(token write, block encode, decompression) of configuration 4, at the nominal
2 % junk and at the junk fraction that brings the overflow pool near its
8192-record limit, and prefill attention over the compressed records beside
decompress-then-attend, at configuration 4's own size and on a small step.

``--impl reference`` runs the CPU pipeline alone (all host threads) as the
reference arm; ``--impl reference-gpu`` and ``--arms`` select single arms;
``--workload`` measures one configuration alone (profiling, experiments).
"""

from __future__ import annotations

import argparse
import atexit
from dataclasses import replace
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

from benchmarks import workloads  # noqa: E402
from fragpack_b200.compression import attn_page as ap  # noqa: E402

METRIC = "decode_attn_effective_logical_kv_bandwidth"
UNIT = "TB/s"
SCALE = 128**-0.5
FALLBACK_HBM_GBS = 6650.0
# Junk fraction of configuration 4 at which fallbacks + spills of the two
# encoded layers land just under the 8192-record overflow pool (seeded run).
NEAR_LIMIT_JUNK = 0.01106
# DRAM traffic of one decode_attn_kernel launch as ncu counted it, kept as text
# beside the other profile summaries: lines of key=value pairs.
TRAFFIC_FILE = ROOT / "profiles" / "decode_attn_kernel_dram_traffic.txt"


def measured_hbm_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


def captured_traffic(workload: str, records_per_launch: float) -> dict | None:
    """DRAM bytes per launch from the ncu capture of ``workload``, scaled by records.

    Every record is read exactly once, so traffic grows in proportion to the
    records a launch reads; the capture is of a reduced batch.
    """
    if not TRAFFIC_FILE.exists():
        return None
    for line in TRAFFIC_FILE.read_text().splitlines():
        if line.startswith("#") or "=" not in line:
            continue
        row = dict(item.split("=", 1) for item in line.split())
        if row.get("workload") != workload:
            continue
        try:
            scale = records_per_launch / float(row["records"])
            return {
                "bytes": (float(row["dram_bytes_read"]) + float(row["dram_bytes_write"])) * scale,
                "source": f"profiles/{TRAFFIC_FILE.name}: capture of {row['records']} records scaled "
                          f"by {scale:.3f}",
            }
        except (KeyError, ValueError, ZeroDivisionError):
            return None
    return None


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
        if self._begin is None:
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
            "window": "from the first warm-up step of the headline to its last end-to-end step",
        }


# --------------------------------------------------------------------------
# CPU pipeline (oracle codec + torch fp32 attention): baseline and reference arm
# --------------------------------------------------------------------------
def host_threads() -> int:
    """Host cores this process may use (a launcher's OMP_NUM_THREADS=1 is not a limit)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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

    threads = oracle.set_threads(host_threads())
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    for _ in range(repeats):
        dec = oracle.decode_records(sample["records"], sample["lens"], sample["tables"], sample["kv"])
        f32 = torch.from_numpy(oracle.bf16_bits_to_f32(dec))  # [n,128,128]
        for (k0, k1, v0, v1, tokens), q in zip(sample["ranges"], sample["q"]):
            k = f32[k0:k1].reshape(-1, 128)[:tokens]
            v = f32[v0:v1].reshape(-1, 128)[:tokens]
            oracle.attention_fp32(q, k, v, SCALE)
    seconds = (time.perf_counter() - t0) / repeats
    return seconds, float(sample["logical_bytes"]), threads


def sample_for_cpu(work: workloads.DecodeWorkload, layers: int, seqs: int, heads: int) -> dict:
    """Copy the records of ``layers`` x ``seqs`` sequences x ``heads`` KV heads to the host."""
    store, cfg = work.store, work.cfg
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
        "what": f"{layers} layer(s) x {seqs} sequence(s) x {heads} KV head(s) of {cfg.name}",
    }


# --------------------------------------------------------------------------
# GPU arms
# --------------------------------------------------------------------------
def validate(work, queries, outputs, layer: int) -> dict:
    """Errors of ``outputs[layer]`` vs fp32 attention over the kept source KV.

    The stated bar (1e-2 max-abs, 2e-3 mean-abs on BF16 outputs) is absolute.
    It is applied as stated to every output of magnitude up to 1.  An output
    of larger magnitude x (the x64 heavy tails of configuration 3 reach ~100)
    is a BF16 number whose own rounding step is up to x * 2^-8 (3.9e-3 x), so
    those are bounded relative to x: 1e-2 for the worst element, 4e-3 (one
    rounding step) for the mean.  Both sets are reported and both must pass.
    """
    cfg = work.cfg
    small, large = [], []
    for (lay, b), kv in work.sample.items():
        if lay != layer:
            continue
        k = kv[0].float()  # [T, H, 128]
        v = kv[1].float()
        for h in range(cfg.kv_heads):
            q = queries[layer][b, h * cfg.group : (h + 1) * cfg.group].float()
            ref = torch.softmax(q @ k[:, h].T * SCALE, -1) @ v[:, h]
            err = (outputs[layer][b, h * cfg.group : (h + 1) * cfg.group].float() - ref).abs()
            big = ref.abs() > 1.0
            small.append(err[~big])
            large.append((err / ref.abs().clamp(min=1.0))[big])
    small, large = torch.cat(small), torch.cat(large)
    nan = bool(torch.isnan(small).any() or torch.isnan(large).any())
    return {
        "max_abs": float(small.max()) if small.numel() else 0.0,
        "mean_abs": float(small.mean()) if small.numel() else 0.0,
        "max_rel_above_1": float(large.max()) if large.numel() else 0.0,
        "mean_rel_above_1": float(large.mean()) if large.numel() else 0.0,
        "outputs_above_1": int(large.numel()),
        "nan": nan,
    }


def merge_validation(a: dict | None, b: dict) -> dict:
    if a is None:
        return dict(b)
    out = {k: max(a[k], b[k]) for k in ("max_abs", "mean_abs", "max_rel_above_1", "mean_rel_above_1")}
    out["outputs_above_1"] = a["outputs_above_1"] + b["outputs_above_1"]
    out["nan"] = a["nan"] or b["nan"]
    return out


def validation_ok(v: dict) -> bool:
    return (not v["nan"] and v["max_abs"] <= 1e-2 and v["mean_abs"] <= 2e-3
            and v["max_rel_above_1"] <= 1e-2 and v["mean_rel_above_1"] <= 4e-3)


class Env:
    """Process placement: one rank per GPU."""

    def __init__(self) -> None:
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.device = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.dist is None:
            return value
        t = torch.tensor([value], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self) -> None:
        if self.dist is not None:
            self.dist.destroy_process_group()


def reference_decode(ref_mod):
    """The reference's host wrapper around its own kernels (fused_attn_decode.py:105-171)."""

    def call(q, tabs, block_table, seq_lens, scale, units, out, ws, replan):
        # Its kernel attends 8 query heads per KV head; smaller groups run
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

    return call


def run_decode(args, env: Env, name: str, arms: list[str], clocks: ClockSampler | None,
               layers_arg: int = 0, cpu_baseline: bool = False) -> dict:
    """Build one decode workload on this rank's shard and measure the listed arms.

    The first arm is the one whose numbers head the result (``value``,
    ``roofline``, ``e2e``); all arms are then timed with interleaved rounds.
    """
    from fragpack_b200.ops.fused_attn_decode import (
        RecordTables,
        decode_attention,
        decode_status,
        decode_units,
        plain_decode_attention,
        workspace_elems,
    )

    world, rank, device, dist = env.world, env.rank, env.device, env.dist
    cfg = workloads.CONFIGS[name]
    if args.batch or args.ctx:
        # Reduced copies of a configuration, for profiler captures.
        ctx = args.ctx or cfg.ctx_max
        cfg = replace(cfg, name=f"{cfg.name}-reduced", batch=args.batch or cfg.batch,
                      ctx_min=min(cfg.ctx_min, ctx), ctx_max=ctx)
    if cfg.kv_heads % world:
        raise SystemExit(f"{world} GPUs do not divide {cfg.kv_heads} KV heads")
    per = cfg.kv_heads // world
    notes = []
    if world == 1 and args.shard_of > 1:
        # One GPU runs what one rank of an N-way KV-head split would (no gather).
        if cfg.kv_heads % args.shard_of:
            raise SystemExit(f"{args.shard_of} shards do not divide {cfg.kv_heads} KV heads")
        per = cfg.kv_heads // args.shard_of
        cfg = replace(cfg, name=f"{cfg.name}-shard-of-{args.shard_of}")
        notes.append(f"one rank's shard of a {args.shard_of}-way KV-head split, without the gather")
    head_slice = slice(rank * per, (rank + 1) * per)
    ref_mod = None
    arms = list(arms)
    if "reference" in arms:
        from oracle import build_ref_kernels

        try:
            ref_mod = build_ref_kernels.module()
        except Exception as exc:  # noqa: BLE001
            if arms[0] == "reference":
                if rank == 0:
                    print(json.dumps({"impl": "reference-gpu",
                                      "unavailable": f"the reference's CUDA extension is not built here: {exc}"}))
                raise SystemExit(0)
            arms = [a for a in arms if a != "reference"]
            notes.append(f"reference kernel arm left out: {exc}")
    if world > 1:
        arms = arms[:1]

    # Resident layers: all of them when they fit, else as many as the budget holds.
    pages_per_layer = cfg.batch * ((cfg.ctx_max + 127) // 128) * 2 * per
    per_layer = pages_per_layer * (ap.DENSE_BYTES + 1280)
    if "plain" in arms:
        per_layer += pages_per_layer * ap.RAW_RECORD_BYTES
    budget = int(args.hbm_budget_gb * 2**30)
    layers = layers_arg or max(1, min(cfg.layers, budget // max(per_layer, 1)))
    if world > 1 and layers > 2:
        # An even count keeps the two gathered copies alternating inside a replayed graph.
        layers -= layers % 2
    work = {}
    for arm in arms:
        key = "plain" if arm == "plain" else "coded"
        if key not in work:
            work[key] = workloads.build_decode_workload(
                cfg, device, seed=args.seed, layers=layers, head_slice=head_slice,
                keep_layers=(0, layers - 1), plain=key == "plain",
            )
    first = work["plain" if arms[0] == "plain" else "coded"]
    built = first.cfg
    B, H, G = built.batch, built.kv_heads, built.group
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    gen = torch.Generator(device=device).manual_seed(args.seed + 100 + rank)
    # One tensor for all layers' queries and one per arm for their outputs, so
    # that the end-to-end step moves each with a single copy.
    q_all = torch.randn(layers, B, H * G, 128, generator=gen, device=device).to(torch.bfloat16)
    queries = [q_all[layer] for layer in range(layers)]

    class Arm:
        pass

    state: dict[str, Arm] = {}
    for arm in arms:
        a = Arm()
        a.work = work["plain" if arm == "plain" else "coded"]
        a.units = decode_units(B, H, sms)
        if arm == "reference":
            # The reference reserves one wave of split capacity (fused_attn_decode.py:58-85).
            a.units = B + max(1, (2 * sms) // H) - 1
        sizes = workspace_elems(H, a.units)
        a.ws = (torch.empty(sizes[0], device=device), torch.empty(sizes[1], device=device),
                torch.empty(sizes[2], dtype=torch.int32, device=device))
        a.out_all = torch.full_like(q_all, float("nan"))
        a.outputs = [a.out_all[layer] for layer in range(layers)]
        a.tabs = [RecordTables(*a.work.store.layer_tables(layer)) for layer in range(layers)]
        a.call = {"fused": decode_attention, "plain": plain_decode_attention}.get(arm)
        if arm == "reference":
            a.call = reference_decode(ref_mod)
        a.graph = None
        state[arm] = a
    lead = state[arms[0]]

    gather = peer_gather = None
    if world > 1 and arms[0] == "fused" and args.gather == "peers":
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
    if world > 1:
        from fragpack_b200.ops.tp import HeadGather

        gather = HeadGather(B, H * G, torch.bfloat16, device)

    def make_step(arm: str):
        a = state[arm]

        def attend(layer: int) -> None:
            a.call(queries[layer], a.tabs[layer], a.work.block_table, a.work.seq_lens, SCALE,
                   a.units, a.outputs[layer], a.ws, replan=layer == 0)

        def step() -> None:
            for layer in range(layers):
                if peer_gather is not None:
                    peer_gather.decode(queries[layer], a.tabs[layer], a.work.block_table,
                                       a.work.seq_lens, SCALE, a.units, a.ws, replan=layer == 0)
                    continue
                attend(layer)
                if gather is not None:
                    # Per-head outputs -> o_proj input layout [B, Hq, 128] on every rank.
                    gather(a.outputs[layer])

        return attend, step

    def statuses() -> int:
        """Status words of this library's arms, OR-ed over the ranks (synchronises)."""
        word = 0
        for arm in arms:
            if arm != "reference":
                word |= decode_status(state[arm].ws, state[arm].units)
        if peer_gather is not None:
            word |= peer_gather.status() << 8
        return int(env.max_over_ranks(float(word)))

    # ---- Correctness gate before any timing: outputs start as NaN.
    checks = {}
    gather_check = None
    for arm in arms:
        a = state[arm]
        attend, step = make_step(arm)
        a.attend, a.step = attend, step
        step()
        torch.cuda.synchronize()
        if peer_gather is not None:
            if peer_gather.status():
                raise SystemExit("a peer did not arrive within the wait limit")
            # The gathered copy of the last layer against an NCCL all-gather of
            # the ranks' own outputs: every rank's heads must sit where o_proj
            # expects them, bit for bit, on every rank.
            got = peer_gather.gathered[(layers - 1) & 1].clone()
            attend(layers - 1)
            want = gather(a.outputs[layers - 1])
            same = torch.tensor([int(torch.equal(got, want))], device=device)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            gather_check = {"bit_equal_with_nccl_all_gather_on_every_rank": bool(same.item()),
                            "rows": int(want.shape[0]), "heads": int(want.shape[1])}
            if not gather_check["bit_equal_with_nccl_all_gather_on_every_rank"] and not args.skip_validation:
                raise SystemExit("peer-gathered outputs differ from the NCCL all-gather")
            if layers > 1:
                attend(0)  # the local copies of the validated layers
            torch.cuda.synchronize()
        result = None
        for layer in sorted({0, layers - 1}):
            result = merge_validation(result, validate(a.work, queries, a.outputs, layer))
        checks[arm] = result
        if not validation_ok(result) and not args.skip_validation:
            raise SystemExit(f"validation of the {arm} arm failed: {result}")
    if statuses():
        raise SystemExit("a bounded device-side wait ran out during validation")

    # ---- CUDA graphs of one step per arm.  NCCL calls stay out of the graph;
    # the peer-store gather is plain kernels (an even number of calls per
    # replay keeps its two copies alternating).
    use_graph = not args.no_graph and (world == 1 or (peer_gather is not None and layers % 2 == 0))
    if use_graph:
        for arm in arms:
            a = state[arm]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                a.step()
            torch.cuda.current_stream().wait_stream(side)
            a.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(a.graph, stream=side):
                a.step()
    # Every rank has captured before any rank replays (a replay's peer wait is bounded).
    env.barrier()

    def run_step(arm: str) -> None:
        a = state[arm]
        if a.graph is not None:
            a.graph.replay()
        else:
            a.step()

    # ---- Headline: warm up (at least W steps and 100 ms), then exactly K steps
    # in one bracket; an event after every step gives the per-step samples.
    if clocks is not None:
        clocks.mark_begin()
    warm = max(args.warmup, 3)
    t0 = time.perf_counter()
    done = 0
    while done < warm or (world == 1 and time.perf_counter() - t0 < 0.1):
        run_step(arms[0])
        done += 1
        if done % 8 == 0:
            torch.cuda.synchronize()
    env.barrier()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    marks[0].record()
    for i in range(args.steps):
        run_step(arms[0])
        marks[i + 1].record()
    env.barrier()
    ms = env.max_over_ranks(marks[0].elapsed_time(marks[-1]))
    ms_per_step = ms / args.steps
    step_samples = [marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps)]
    status_after_timing = statuses()

    # ---- All arms, interleaved rounds (the template of the reference's step
    # benchmark): each round times a short burst of every arm in turn.
    compare = {}
    if len(arms) > 1:
        burst = max(1, int(np.ceil(25.0 / max(ms_per_step, 1e-3))))
        rounds = 20
        samples = {arm: [] for arm in arms}
        pairs = []
        for _ in range(rounds):
            for arm in arms:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(burst):
                    run_step(arm)
                e1.record()
                pairs.append((arm, e0, e1))
        torch.cuda.synchronize()
        for arm, e0, e1 in pairs:
            samples[arm].append(e0.elapsed_time(e1) / burst)
        for arm in arms:
            med = float(np.median(samples[arm]))
            compare[arm] = {
                "us_per_layer": med * 1e3 / layers,
                "us_per_layer_min": float(np.min(samples[arm])) * 1e3 / layers,
                "rounds": rounds,
                "steps_per_round": burst,
                "validation": checks[arm],
            }
        for arm in arms[1:]:
            compare[arm]["fused_speedup"] = compare[arm]["us_per_layer"] / compare[arms[0]]["us_per_layer"]

    # ---- Eager launches (no graph): one event per decode call on the launching
    # stream, for the per-launch duration of the dominant kernel.
    eager_call_ms = None
    if peer_gather is None:
        per_call = []
        for _ in range(3):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(layers + 1)]
            lead.attend(0)
            evs[0].record()
            for layer in range(layers):
                lead.call(queries[layer], lead.tabs[layer], lead.work.block_table, lead.work.seq_lens,
                          SCALE, lead.units, lead.outputs[layer], lead.ws, replan=False)
                evs[layer + 1].record()
            torch.cuda.synchronize()
            per_call.append(np.mean([evs[i].elapsed_time(evs[i + 1]) for i in range(layers)]))
        eager_call_ms = float(np.min(per_call))
    call_ms = eager_call_ms if eager_call_ms is not None else ms_per_step / layers
    if use_graph:
        # Eager calls are paced by the host (one ctypes call per layer), so their
        # event spacing includes host gaps.  Inside the replayed graph a layer is
        # exactly the attention kernel followed by the small merge kernel: use
        # that time (an upper bound on the attention kernel's own duration).
        call_ms = min(call_ms, ms_per_step / layers)

    # ---- End to end through the public API with host buffers.
    q_host = q_all.cpu().pin_memory()
    out_host = torch.empty_like(q_all, device="cpu").pin_memory()
    bt_host = lead.work.block_table.cpu().pin_memory()
    len_host = lead.work.seq_lens.cpu().pin_memory()
    h2d = q_host.numel() * 2 + bt_host.numel() * 4 + len_host.numel() * 4
    d2h = out_host.numel() * 2

    def e2e_step() -> None:
        lead.work.block_table.copy_(bt_host, non_blocking=True)
        lead.work.seq_lens.copy_(len_host, non_blocking=True)
        q_all.copy_(q_host, non_blocking=True)
        run_step(arms[0])
        if peer_gather is not None:
            # The result lives in the two gathered copies (the last two layers');
            # read this rank's heads of each back, the same bytes per layer.
            lo = rank * H * G
            for layer in range(layers):
                out_host[layer].copy_(peer_gather.gathered[layer & 1][:, lo : lo + H * G], non_blocking=True)
        else:
            out_host.copy_(lead.out_all, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(3, min(args.steps, int(np.ceil(500.0 / max(ms_per_step, 1e-3)))))
    for _ in range(3):
        e2e_step()
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    env.barrier()
    e2e_ms = env.max_over_ranks((time.perf_counter() - t0) * 1e3 / e2e_steps)
    status_after_e2e = statuses()
    if clocks is not None:
        clocks.mark_end()
    if (status_after_timing or status_after_e2e) and not args.skip_validation:
        raise SystemExit(f"a bounded device-side wait ran out during the timed steps "
                         f"(status {status_after_timing:#x} / {status_after_e2e:#x}): the step times are invalid")
    final = validate(lead.work, queries, lead.outputs, layers - 1) if peer_gather is None else None
    if final is not None and not validation_ok(final) and not args.skip_validation:
        raise SystemExit(f"outputs after the timed steps fail validation: {final}")

    logical_all = lead.work.logical_bytes * layers * world  # every rank holds an equal head shard
    stored_layer = float(np.mean(lead.work.compressed_bytes))
    records_layer = float(int(((lead.work.lens_host + 127) // 128).sum()) * 2 * H)
    peak, peak_kind = measured_hbm_peak()
    achieved = stored_layer / (call_ms * 1e-3) / 1e9
    traffic = captured_traffic(name, records_layer) if arms[0] == "fused" else None
    arm_text = {
        "fused": "fused decode over compressed records",
        "plain": "plain BF16 records, no decode step (comparison)",
        "reference": "the reference's CUDA kernels built for sm_100a, reading this library's records (comparison)",
    }
    kernel_name = {"fused": "decode_attn_kernel", "plain": "plain_attn_kernel",
                   "reference": "reference decode_attn"}[arms[0]]
    line = {
        "metric": METRIC,
        "value": logical_all / (ms_per_step * 1e-3) / 1e12,
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": done,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16 KV and P, fp32 softmax/accumulate; u8/u32 integer decode",
        "data": "synthetic (seeded per-channel lognormal-scaled Gaussian BF16 KV, K outlier channels)",
        "config": {
            "workload": cfg.name,
            "arm": arm_text[arms[0]],
            "layers_resident": layers,
            "layers_model": cfg.layers,
            "kv_heads_per_gpu": H,
            "q_heads_per_gpu": H * G,
            "batch": B,
            "context": [int(lead.work.lens_host.min()), int(lead.work.lens_host.max())],
            "parallelism": f"kv-head shard tp{world}" + (
                "" if world == 1 else
                " + output gather by the merge kernel (peer stores over NVLink)" if peer_gather is not None
                else " + NCCL all-gather per layer"),
            "cuda_graph": bool(use_graph),
            "l2_policy": "inputs larger than L2: every layer reads distinct pages, "
                         f"{stored_layer * layers / 2**20:.0f} MiB per step vs 126 MiB L2",
        },
        "us_per_layer": ms_per_step * 1e3 / layers,
        "us_per_layer_median": float(np.median(step_samples)) * 1e3 / layers,
        "step_ms_samples": [round(x, 4) for x in step_samples[:64]],
        "eager_us_per_layer": None if eager_call_ms is None else eager_call_ms * 1e3,
        "kv_ratio": lead.work.logical_bytes / stored_layer,
        "compressed_gbs": stored_layer * layers * world / (ms_per_step * 1e-3) / 1e9,
        "e2e": {
            "value": logical_all / (e2e_ms * 1e-3) / 1e12,
            "unit": UNIT,
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "ms_per_step": e2e_ms,
            "steps": e2e_steps,
        },
        # This library's kernels per step: one planner, then attention + merge
        # per layer (+ the two arrival kernels of the peer gather).
        "gpu_launches": 0 if arms[0] == "reference"
        else args.steps * (1 + (4 if peer_gather is not None else 2) * layers),
        "roofline": {
            "bound": "hbm",
            "kernel": kernel_name + " (duration includes the merge kernel that follows it)",
            "achieved": achieved,
            "peak": peak,
            "peak_kind": peak_kind,
            "unit": "GB/s",
            "frac": achieved / peak,
            "traffic": traffic["bytes"] if traffic else None,
            "traffic_source": traffic["source"] if traffic else None,
            "algorithmic_bytes_per_launch": stored_layer,
            "launch_ms": call_ms,
        },
        "validation": checks[arms[0]],
        "status_words": {"after_timed_steps": status_after_timing, "after_e2e_steps": status_after_e2e},
    }
    if gather_check is not None:
        line["gather_check"] = gather_check
    if compare:
        line["arms"] = compare
    if notes:
        line["notes"] = notes
    if cpu_baseline and rank == 0 and world == 1:
        sample = sample_for_cpu(work["coded"], layers=1, seqs=min(B, args.cpu_seqs),
                                heads=min(H, args.cpu_heads))
        first_pass, logical, threads = cpu_pipeline(sample)
        passes = max(1, int(np.ceil(args.cpu_seconds / max(first_pass, 1e-3))))
        seconds, logical, threads = cpu_pipeline(sample, repeats=passes)
        line["cpu_baseline"] = {
            "value": logical / seconds / 1e12,
            "unit": UNIT,
            "cores": threads,
            "kind": "port",
            "sample": sample["what"] + f" ({len(sample['lens'])} records; {passes} timed passes of "
                      f"{seconds:.2f} s each after one warm-up pass)",
        }
    del state, work, lead
    torch.cuda.empty_cache()
    return line


def run_codec(args, junk: float, layers: int = 2, steps: int | None = None) -> dict:
    """Prefill side (configuration 4): token write + block encode, then decompression.

    One step = one layer of the MHA stress geometry (32 KV heads, 16 x 8192
    tokens = 1024 blocks): the tokens are scattered into staging, every completed
    block is encoded into its arena page, and all blocks are decompressed into the
    BF16 workspace.  Each phase is timed with CUDA events on its own.
    """
    from benchmarks import synth
    from fragpack_b200.compression.attn_tables import device_tables
    from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    cfg = workloads.CONFIGS["c4"]
    heads = cfg.kv_heads
    steps = steps or args.codec_steps
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
    first_counters = None
    for it in range(2 + steps):
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
            if it >= 2:
                for name, a, b in (("write", 0, 1), ("encode", 1, 2), ("gather", 2, 3)):
                    times[name].append(ev[a].elapsed_time(ev[b]))
            if it == 0:
                # Bit-exact reconstruction of what was written (a record dropped
                # because the overflow pool is full stays readable in staging
                # until its slot is reused).
                src_k = kv[layer][0].view(blocks, 128, heads, 128)
                src_v = kv[layer][1].view(blocks, 128, heads, 128)
                ok &= bool(torch.equal(wk, src_k)) and bool(torch.equal(wv, src_v))
        store.commit()
        if it == 0:
            first_counters = store.counters.cpu().numpy().copy()
    records = blocks * 2 * heads
    rec_bytes = float((store.rec_len[0, ids_dev.long()].to(torch.int64) + ap.DENSE_BYTES).sum().item())
    peak, peak_kind = measured_hbm_peak()
    ms = {k: float(np.median(v)) for k, v in times.items()}
    enc_bytes = records * 32768 + rec_bytes
    dec_bytes = rec_bytes + records * 32768
    c = first_counters
    out = {
        "workload": cfg.name,
        "junk_fraction": junk,
        "layers_resident": layers,
        "kv_heads": heads,
        "tokens_per_layer": tokens,
        "records_per_layer": records,
        "overflow_records": args.overflow,
        "timed_layer_passes": len(times["encode"]),
        "bit_exact_roundtrip": ok,
        "mean_record_bytes": rec_bytes / records,
        # One pass over all layers (the state the pool limit is about).
        "one_pass_counters": {"encoded": int(c[7]), "fallbacks": int(c[6]), "spills": int(c[8]),
                              "overflow_records_wanted_vs_pool": float(int(c[6]) / max(args.overflow, 1)),
                              "err_overflow": int(c[5]), "err_staging": int(c[4])},
        "write": {"ms_per_layer": ms["write"],
                  "GBps": (records * 32768 * 2) / (ms["write"] * 1e-3) / 1e9,
                  "roofline_frac": (records * 32768 * 2) / (ms["write"] * 1e-3) / 1e9 / peak},
        "encode": {"ms_per_layer": ms["encode"], "GBps": enc_bytes / (ms["encode"] * 1e-3) / 1e9,
                   "roofline_frac": enc_bytes / (ms["encode"] * 1e-3) / 1e9 / peak},
        "decompress": {"ms_per_layer": ms["gather"], "GBps": dec_bytes / (ms["gather"] * 1e-3) / 1e9,
                       "roofline_frac": dec_bytes / (ms["gather"] * 1e-3) / 1e9 / peak},
        "peak": peak, "peak_kind": peak_kind,
    }
    del store, arenas, kv, wk, wv
    torch.cuda.empty_cache()
    return out


def run_prefill_attention(args, requests: int = 4, cached: int = 2048, chunk: int = 512) -> dict:
    """Prefill attention of a chunk over cached context, MHA geometry of configuration 4.

    ``requests`` sequences hold ``cached + chunk`` tokens in the store (32 KV
    heads, group 1, junk-free values: junk bit patterns overflow fp32 attention
    in any implementation); the last ``chunk`` tokens of each are the queries.
    Two paths over the same store: the fused kernel (records decoded into
    tensor-core operand tiles, nothing written back) and the reference's two
    steps (decompress into the BF16 workspace, then attention over it - torch
    SDPA per request where the reference calls FlashAttention-3).
    """
    from fragpack_b200.integrations.vllm.backend import plan_prefill_groups, workspace_prefill_attention
    from fragpack_b200.ops.fused_attn_decode import RecordTables
    from fragpack_b200.ops.prefill_attn import prefill_attention, prefill_status

    device = torch.device("cuda", 0)
    total = cached + chunk
    cfg = replace(workloads.CONFIGS["c4"], name="c4-mha-chunked-prefill", batch=requests, ctx_min=total,
                  ctx_max=total, junk=0.0)
    work = workloads.build_decode_workload(cfg, device, seed=args.seed, layers=1, keep_layers=(0,), keep_seqs=1)
    H, G = work.cfg.kv_heads, work.cfg.group
    gen = torch.Generator(device=device).manual_seed(args.seed + 9)
    q = torch.randn(requests * chunk, H * G, 128, generator=gen, device=device).to(torch.bfloat16)
    tabs = RecordTables(*work.store.layer_tables(0))
    q_start = torch.arange(0, requests * chunk + 1, chunk, dtype=torch.int32, device=device)
    ctx_lens = torch.full((requests,), total, dtype=torch.int32, device=device)
    out_fused = torch.full_like(q, float("nan"))
    out_two = torch.full_like(q, float("nan"))
    pages = total // 128
    wk = torch.empty(requests * pages, 128, H, 128, dtype=torch.bfloat16, device=device)
    wv = torch.empty_like(wk)
    qsl = np.arange(0, requests * chunk + 1, chunk, dtype=np.int64)
    seq = np.full(requests, total, np.int64)
    group = plan_prefill_groups(work.block_table, 0, requests, qsl, seq, requests * pages, device)[0]

    def fused() -> None:
        prefill_attention(q, tabs, work.block_table, q_start, ctx_lens, SCALE, out_fused, chunk)

    def two_step() -> None:
        work.store.gather(0, group.src_blocks, wk, wv)
        workspace_prefill_attention(q, wk, wv, group, SCALE, out_two)

    def timed(fn, rounds: int) -> list[float]:
        fn()
        torch.cuda.synchronize()
        samples = []
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            samples.append(e0.elapsed_time(e1))
        return samples

    t_fused, t_two = timed(fused, 10), timed(two_step, 5)
    status = prefill_status(device)
    # fp32 causal attention over the kept source KV of request 0.
    kv = work.sample[(0, 0)].float()
    mask = torch.ones(chunk, total, dtype=torch.bool, device=device).tril(total - chunk)
    small, large = [], []
    for h in range(0, H, max(1, H // 4)):
        s = (q[:chunk, h].float() @ kv[0][:, h].T) * SCALE
        ref = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ kv[1][:, h]
        err = (out_fused[:chunk, h].float() - ref).abs()
        big = ref.abs() > 1.0
        small.append(err[~big])
        large.append((err / ref.abs().clamp(min=1.0))[big])
    small, large = torch.cat(small), torch.cat(large)
    # Query i sees cached + i + 1 keys: 4 flops per (query, key, dim) for the two products.
    flops = 4.0 * requests * H * G * 128 * (chunk * cached + chunk * (chunk + 1) / 2)
    med_fused, med_two = float(np.median(t_fused)), float(np.median(t_two))
    out = {
        "workload": f"{cfg.name}: {requests} requests x ({cached} cached + {chunk} new tokens), "
                    f"{H} KV heads, group {G}, one layer",
        "fused_over_records": {"ms_per_layer": med_fused, "tflops": flops / (med_fused * 1e-3) / 1e12,
                               "kernel": "prefill_attn_kernel (tcgen05, operands decoded in shared memory)"},
        "decompress_then_attend": {"ms_per_layer": med_two, "tflops": flops / (med_two * 1e-3) / 1e12,
                                   "kernels": "gather_kernel + torch SDPA per request"},
        "speedup": med_two / med_fused,
        "validation_vs_fp32_reference": {
            "max_abs": float(small.max()), "mean_abs": float(small.mean()),
            "max_rel_above_1": float(large.max()) if large.numel() else 0.0,
            "mean_rel_above_1": float(large.mean()) if large.numel() else 0.0,
            "outputs_above_1": int(large.numel())},
        "max_abs_between_paths": float((out_fused.float() - out_two.float()).abs().max()),
        "status_word": status,
    }
    del work, wk, wv
    torch.cuda.empty_cache()
    return out


def brief(line: dict) -> dict:
    """The part of a decode result that the headline line carries for an extra workload."""
    keep = ("us_per_layer", "us_per_layer_median", "eager_us_per_layer", "value", "kv_ratio", "validation")
    out = {k: line[k] for k in keep if k in line}
    out["workload"] = line["config"]["workload"]
    out["layers_resident"] = line["config"]["layers_resident"]
    out["cuda_graph"] = line["config"]["cuda_graph"]
    out["steps"] = line["steps"]
    out["roofline_frac"] = line["roofline"]["frac"]
    out["compressed_GBps"] = line["roofline"]["achieved"]
    out["e2e_value"] = line["e2e"]["value"]
    if "arms" in line:
        out["arms"] = {k: {x: v[x] for x in ("us_per_layer", "fused_speedup") if x in v}
                       for k, v in line["arms"].items()}
    return out


def run_ours(args) -> dict:
    env = Env()
    clocks = ClockSampler(env.local).start()
    arms = [a.strip() for a in args.arms.split(",") if a.strip()]
    if args.impl == "reference-gpu":
        arms = ["reference"]
    if args.workload == "c4":
        line = run_codec(args, args.junk if args.junk >= 0 else NEAR_LIMIT_JUNK, args.layers or 2)
        line.update({"metric": "block_encode_and_decompress_throughput", "n_gpus": 1})
        if args.prefill_attention:
            shape = [int(x) for x in args.prefill_shape.split(",")]
            line["prefill_attention"] = run_prefill_attention(args, *shape)
        clocks.stop()
        env.close()
        return line
    name = args.workload or "c5"
    line = run_decode(args, env, name, arms, clocks, layers_arg=args.layers,
                      cpu_baseline=not args.no_cpu_baseline and arms[0] == "fused")
    clocks.stop()
    line["clocks"] = clocks.summary()
    if args.impl == "reference-gpu":
        line["impl"] = "reference-gpu"
    if env.world == 1 and env.rank == 0 and not args.workload and not args.no_extras and arms[0] == "fused":
        # The other configurations, in this same process (steps sized to about
        # half a second per timed region).
        extra = {}
        keep = (args.steps, args.warmup)
        for other, steps in (("c2", 500), ("c3", 100)):
            args.steps, args.warmup = steps, 20
            extra[other] = brief(run_decode(args, env, other, arms, None))
        args.steps, args.warmup = keep
        extra["c4_prefill_as_written_junk_2pct"] = run_codec(args, 0.02)
        extra["c4_prefill_near_overflow_limit"] = run_codec(args, NEAR_LIMIT_JUNK)
        # Configuration 4's own size (16 requests of 8192 tokens: the last 2048-token
        # chunk over 6144 cached tokens), and a small chunked-prefill step.
        extra["c4_prefill_attention"] = run_prefill_attention(args, requests=16, cached=6144, chunk=2048)
        extra["c4_prefill_attention_small"] = run_prefill_attention(args)
        line["extra"] = extra
    env.close()
    return line if env.rank == 0 else {}


def run_reference(args) -> dict:
    """Reference arm: the CPU codec (oracle port) + torch CPU fp32 attention."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return {}
    import oracle
    from benchmarks import synth

    name = args.workload or "c5"
    cfg = workloads.CONFIGS[name]
    # Bounded sample of the workload: one layer, a few (sequence, head) pairs
    # at the configuration's own context length.
    rng = np.random.default_rng(args.seed)
    scales = synth.channel_scales(args.seed + 1, 1, cfg.kv_heads)[0]
    tokens = cfg.ctx_max
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
    oracle.set_threads(host_threads())
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
    what = (f"{pairs} (sequence, KV head) pairs x {tokens} tokens of one layer of {cfg.name} per step "
            f"({len(lens)} records), {threads} host threads (set explicitly)")
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
        "scaling": "strong",
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
    parser.add_argument("--steps", type=int, default=0,
                        help="timed steps (default: 100 for the GPU arms, 3 for --impl reference)")
    parser.add_argument("--warmup", type=int, default=-1,
                        help="warm-up steps (default: 10 for the GPU arms, 1 for --impl reference)")
    parser.add_argument("--impl", choices=("ours", "reference", "reference-gpu"), default="ours",
                        help="reference: the CPU codec + attention (the reference arm); reference-gpu: the "
                             "reference's own CUDA kernels built for sm_100a alone (1 GPU)")
    parser.add_argument("--workload", choices=("c2", "c3", "c4", "c5"), default=None,
                        help="measure one configuration alone (default: c5 headline + the others as extras)")
    parser.add_argument("--arms", default="fused,reference,plain",
                        help="arms timed in this process, the first one heads the line: fused, reference "
                             "(the reference's CUDA kernels), plain (BF16 records, no decode step)")
    parser.add_argument("--junk", type=float, default=-1.0, help="c4: junk fraction")
    parser.add_argument("--overflow", type=int, default=8192, help="c4: overflow records")
    parser.add_argument("--codec-steps", type=int, default=5, help="c4: timed passes over the layers")
    parser.add_argument("--prefill-attention", action="store_true",
                        help="c4: also time prefill attention over compressed records")
    parser.add_argument("--prefill-shape", default="4,2048,512",
                        help="c4 --prefill-attention: requests,cached tokens,new tokens")
    parser.add_argument("--gather", choices=("peers", "nccl"), default="peers",
                        help="N > 1: how the per-rank outputs reach every rank's o_proj input")
    parser.add_argument("--layers", type=int, default=0, help="resident layers (default: what fits)")
    parser.add_argument("--hbm-budget-gb", type=float, default=60.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--batch", type=int, default=0, help="override the batch (profiling)")
    parser.add_argument("--ctx", type=int, default=0, help="override the context (profiling)")
    parser.add_argument("--shard-of", type=int, default=0,
                        help="one GPU: measure one rank's head shard of an N-way split (profiling)")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--no-extras", action="store_true", help="headline workload only")
    parser.add_argument("--skip-validation", action="store_true",
                        help="keep going when the correctness gate fails (kernel experiments only)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--cpu-seqs", type=int, default=1)
    parser.add_argument("--cpu-heads", type=int, default=8)
    parser.add_argument("--cpu-pairs", type=int, default=8,
                        help="reference arm: (sequence, KV head) pairs decoded and attended per step")
    parser.add_argument("--cpu-seconds", type=float, default=12.0,
                        help="CPU baseline: seconds of host work to time")
    args = parser.parse_args()
    if args.impl == "reference":
        args.steps = args.steps or 3
        args.warmup = args.warmup if args.warmup >= 0 else 1
        line = run_reference(args)
    else:
        args.steps = args.steps or 100
        args.warmup = args.warmup if args.warmup >= 0 else 10
        line = run_ours(args)
    if line:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
