#!/usr/bin/env python
"""Benchmark of the decode-time KV-cache hot path on B200.

A step is one decode step of the B=32 x 4K-context configuration over all 43 layers: per layer, append
each sequence's new latent row into the paged pool, then run the absorbed-MLA decode attention through
the block table (the gather is fused into the attention kernel's TMA loads). The pool (43 x 2048 blocks
x 64 rows x 576 bf16 = 6.49 GB) is resident in HBM; per-layer working sets (151 MB) exceed the L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Under torchrun (N > 1) every rank runs the same per-GPU workload on its own sequences (weak scaling, no
data-path collective: batched decode is partitioned by sequence). Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ascend-moe-engine_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

LAYERS = 43           # overridden by --layers for profiling captures
BATCH = 32
CONTEXT = 4096          # tokens attended per sequence, including the one appended this step
BLOCK = 64
HEADS = 64
ROW = 576
LATENT = 512
SCALE = 1.0 / 24.0      # 1/sqrt(576)
SEED = 20251008
METRIC = "decode attn tokens/s/GPU at B=32x4K ctx (43 layers: KV append + paged absorbed-MLA attention)"

ATTN_BYTES_PER_LAUNCH = BATCH * CONTEXT * ROW * 2 + BATCH * HEADS * ROW * 2 + BATCH * HEADS * LATENT * 2
# DRAM bytes of one decode launch from the committed ncu capture (dram__bytes_read.sum + dram__bytes_write.sum).
NCU_DRAM_BYTES_PER_LAUNCH = 153_830_000 + 4_910_000
ATTN_FLOPS_PER_LAUNCH = BATCH * CONTEXT * HEADS * (ROW + LATENT) * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        median = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": median, "sm_max_mhz": sm_max, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ---------------------------------------------------------------------------------------------------
# CPU reference arm: the oracle (the reference's own operators are closed binaries)
# ---------------------------------------------------------------------------------------------------
class CpuSampler:
    """Times the oracle's append + attention on a bounded sample of the step: `layers` layers x `seqs`
    sequences at the full 4096-token context, all host threads, scaled linearly to the full step."""

    def __init__(self):
        import numpy as np

        import kvo

        self.np, self.kvo = np, kvo
        self.threads = int(kvo.lib().kvo_num_threads())
        self.blocks = CONTEXT // BLOCK
        self._data = {}

    def _inputs(self, seqs: int):
        if seqs not in self._data:
            np, kvo = self.np, self.kvo
            rows = seqs * self.blocks * BLOCK
            pool = kvo.normal_bf16(rows * ROW, kvo.STREAM_KV).reshape(rows, ROW)
            table = kvo.permutation(seqs * self.blocks).reshape(seqs, self.blocks)
            q = kvo.make_q(seqs)
            new = kvo.normal_bf16(seqs * ROW, kvo.STREAM_NEW).reshape(seqs, ROW)
            kv_len = np.full(seqs, CONTEXT, dtype=np.int32)
            slots = (table[:, -1].astype(np.int64) * BLOCK + BLOCK - 1).astype(np.int32)
            self._data[seqs] = (pool, table, q, new, kv_len, slots)
        return self._data[seqs]

    def run(self, seqs: int, layers: int) -> float:
        kvo = self.kvo
        pool, table, q, new, kv_len, slots = self._inputs(seqs)
        t0 = time.perf_counter()
        for _ in range(layers):
            kvo.append(pool, new[:, :LATENT], new[:, LATENT:], slots)
            kvo.mla_decode(q, pool, table, kv_len, BLOCK, SCALE)
        return time.perf_counter() - t0

    def plan(self, target_seconds: float):
        """Chooses (seqs, layers) so that one sample takes about target_seconds."""
        probe_seqs = max(1, min(BATCH, (self.threads + HEADS - 1) // HEADS))
        per_seq_layer = self.run(probe_seqs, 1) / probe_seqs
        seqs = int(max(probe_seqs, min(BATCH, target_seconds / max(per_seq_layer, 1e-9))))
        layers = int(max(1, min(LAYERS, target_seconds / max(per_seq_layer * seqs, 1e-9))))
        return seqs, layers

    def sample(self, seqs: int, layers: int):
        t = self.run(seqs, layers)
        step_seconds = t * (BATCH / seqs) * (LAYERS / layers)
        desc = (f"{layers} of {LAYERS} layers x {seqs} of {BATCH} sequences at context {CONTEXT}, "
                f"{t:.2f} s measured, scaled linearly to the full step")
        return BATCH / step_seconds, desc


def cpu_sample(target_seconds: float = 12.0):
    """One bounded CPU sample. Returns (tokens/s for the full step, description, threads)."""
    sampler = CpuSampler()
    seqs, layers = sampler.plan(target_seconds)
    value, desc = sampler.sample(seqs, layers)
    return value, desc, sampler.threads


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    sampler = CpuSampler()
    # the whole --warmup/--steps run is held to about 100 s of CPU work
    seqs, layers = sampler.plan(max(0.2, min(12.0, 100.0 / max(1, args.warmup + args.steps))))
    values, desc = [], ""
    for i in range(args.warmup + args.steps):
        v, desc = sampler.sample(seqs, layers)
        if i >= args.warmup:
            values.append(v)
    value = sum(values) / len(values)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * BATCH / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[1]: B=32 x ctx 4096, 43 layers, block 64, permuted block tables",
                   "arm": "CPU oracle port of the path (the reference's operators are closed CANN binaries); "
                          "each step is the bounded sample below"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": sampler.threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------------------------------
class Workload:
    """Device-resident state of configs[1] on one GPU."""

    def __init__(self, torch, b200kv, seed_offset: int = 0):
        import numpy as np

        import kvo

        self.torch, self.kv = torch, b200kv
        blocks_per_seq = CONTEXT // BLOCK
        self.blocks = BATCH * blocks_per_seq
        rows = self.blocks * BLOCK
        self.pool = torch.empty((LAYERS, rows, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(self.pool, SEED + seed_offset, kvo.STREAM_KV)
        table = kvo.permutation(self.blocks, seed=SEED + seed_offset).reshape(BATCH, blocks_per_seq)
        self.table_np = table
        self.table = torch.from_numpy(table).cuda()
        self.kv_len = torch.full((BATCH,), CONTEXT, dtype=torch.int32, device="cuda")
        slots = (table[:, -1].astype(np.int64) * BLOCK + (CONTEXT - 1) % BLOCK).astype(np.int32)
        self.slots_np = slots
        self.slots = torch.from_numpy(slots).cuda()
        self.q = torch.empty((LAYERS, BATCH, HEADS, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(self.q, SEED + seed_offset, kvo.STREAM_Q, 0, SCALE)
        self.new_rows = torch.empty((LAYERS, BATCH, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(self.new_rows, SEED + seed_offset, kvo.STREAM_NEW)
        self.out = torch.empty((LAYERS, BATCH, HEADS, LATENT), dtype=torch.bfloat16, device="cuda")
        self.ws = torch.empty(b200kv.decode_workspace_bytes(BATCH, HEADS), dtype=torch.uint8, device="cuda")
        self.status = b200kv.new_status()
        self.views = [b200kv.pool_view(self.pool[layer]) for layer in range(LAYERS)]
        self.launches = 0

    def layer(self, layer: int, q, new_rows, out, variant, stream=None):
        kv = self.kv
        kv.append(self.views[layer], new_rows[:, :LATENT], new_rows[:, LATENT:], self.slots, status=self.status,
                  stream=stream)
        kv.mla_decode(q, self.views[layer], self.table, self.kv_len, BLOCK, SCALE, out=out, workspace=self.ws,
                      variant=variant, status=self.status, stream=stream)
        self.launches += 3  # append, decode, finalize

    def step_resident(self, variant, events=None, fused=False):
        """43 layers of append + attention. fused: the append rides in the attention launch (the decode kernel
        writes each sequence's new row before it reads that tile) instead of a launch of its own."""
        torch = self.torch
        for layer in range(LAYERS):
            new = self.new_rows[layer]
            if not fused:
                self.kv.append(self.views[layer], new[:, :LATENT], new[:, LATENT:], self.slots, status=self.status)
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            self.kv.mla_decode(self.q[layer], self.views[layer], self.table, self.kv_len, BLOCK, SCALE,
                               out=self.out[layer], workspace=self.ws, variant=variant, status=self.status,
                               new_rows=(new[:, :LATENT], new[:, LATENT:]) if fused else None,
                               stable_tables=True)  # table and lengths are uploaded before the step
            if events is not None:
                e1.record()
                events.append((e0, e1))
            self.launches += 2 if fused else 3


def check_against_oracle(torch, b200kv, wl: Workload, variant) -> float:
    """One sequence of one layer, copied back and recomputed by the oracle."""
    import numpy as np

    import kvo

    layer, b = min(7, LAYERS - 1), 5
    wl.step_resident(variant)
    torch.cuda.synchronize()
    rows = (wl.table_np[b].astype(np.int64)[:, None] * BLOCK + np.arange(BLOCK)[None, :]).reshape(-1)
    kv_rows = wl.pool[layer][torch.from_numpy(rows).cuda()].contiguous()
    pool_np = kv_rows.view(torch.int16).cpu().numpy().view(np.uint16)
    q_np = wl.q[layer, b].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)[None]
    table = np.arange(CONTEXT // BLOCK, dtype=np.int32)[None]
    want, _ = kvo.mla_decode(q_np, pool_np, table, np.array([CONTEXT], np.int32), BLOCK, SCALE, use_double=True)
    got = wl.out[layer, b].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    err = float(np.abs(kvo.bf16_to_f32(got) - kvo.bf16_to_f32(want[0])).max())
    if not err <= 2e-3:
        raise RuntimeError(f"bench self-check failed: attention differs from the oracle by {err:.3e}")
    # the appended row is in the pool, bit for bit
    slot = int(wl.slots_np[b])
    if not torch.equal(wl.pool[layer, slot].view(torch.int16), wl.new_rows[layer, b].view(torch.int16)):
        raise RuntimeError("bench self-check failed: appended row not found in the pool")
    return err


def measure_move_kernels(torch, b200kv, wl: Workload, hbm_peak: float, use_graph: bool = True):
    """Bandwidth of the two pure-movement kernels on inputs larger than L2: a prefill-sized append
    (64 sequences x 256 rows, the churn configuration's chunk) and a gather of one full layer."""
    import numpy as np

    rows = 64 * 256
    src = torch.empty((4, rows, ROW), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(src, SEED, 3)
    perm = torch.randperm(wl.blocks * BLOCK, device="cuda", dtype=torch.int64)
    slot_sets = [perm[i * rows:(i + 1) * rows].to(torch.int32).contiguous() for i in range(4)]
    res = {}

    def timeit(fn, iters):
        # `iters` launches captured in one CUDA graph (Python call overhead exceeds these kernels' duration)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(3):
                fn(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if not use_graph:  # profiling captures: a few plain launches (their timing includes Python)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(4):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / 4 * 1e-3
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * iters) * 1e-3

    # Append: rotate over 4 source sets and all 43 layer pools so neither side is L2-resident.
    def do_append(i):
        b200kv.append(wl.views[i % LAYERS], src[i % 4][:, :LATENT], src[i % 4][:, LATENT:], slot_sets[i % 4],
                      status=wl.status)
    t = timeit(do_append, 86)
    bytes_append = rows * (ROW * 2 * 2 + 4)
    res["append"] = {"rows_per_launch": rows, "algorithmic_bytes": bytes_append, "us_per_launch": t * 1e6,
                     "achieved_gbs": bytes_append / t * 1e-9, "frac_of_measured_hbm": bytes_append / t * 1e-9 / hbm_peak}
    # Decode-shaped append (32 rows): launch-latency bound, reported as latency.
    t = timeit(lambda i: b200kv.append(wl.views[i % LAYERS], wl.new_rows[i % LAYERS][:, :LATENT],
                                       wl.new_rows[i % LAYERS][:, LATENT:], wl.slots, status=wl.status), 86)
    res["append_decode_step"] = {"rows_per_launch": BATCH, "us_per_launch": t * 1e6}
    # Gather: every row of one layer (32 x 4096 rows = 151 MB read + 151 MB written).
    total = BATCH * CONTEXT
    out_l = torch.empty((2, total, LATENT), dtype=torch.bfloat16, device="cuda")
    out_r = torch.empty((2, total, 64), dtype=torch.bfloat16, device="cuda")
    offsets = torch.arange(BATCH, dtype=torch.int64, device="cuda") * CONTEXT

    def do_gather(i):
        b200kv.gather(wl.views[i % LAYERS], wl.table, wl.kv_len, BLOCK, out_l[i % 2], out_r[i % 2], offsets, total,
                      status=wl.status)
    t = timeit(do_gather, 43)
    bytes_gather = total * ROW * 2 * 2 + wl.blocks * 4
    res["gather"] = {"rows_per_launch": total, "algorithmic_bytes": bytes_gather, "us_per_launch": t * 1e6,
                     "achieved_gbs": bytes_gather / t * 1e-9, "frac_of_measured_hbm": bytes_gather / t * 1e-9 / hbm_peak}
    # Append of a whole layer's rows (a 32 x 4096-token prefill written in one call, 151 MB read + 151 MB
    # written): the same kernel where its fixed costs (first loads, write drain, about 3 us) are amortised.
    full_slots = perm.to(torch.int32).contiguous()

    def do_append_layer(i):
        b200kv.append(wl.views[i % LAYERS], out_l[i % 2], out_r[i % 2], full_slots, status=wl.status)
    t = timeit(do_append_layer, 43)
    bytes_layer = total * (ROW * 2 * 2 + 4)
    res["append_layer"] = {"rows_per_launch": total, "algorithmic_bytes": bytes_layer, "us_per_launch": t * 1e6,
                           "achieved_gbs": bytes_layer / t * 1e-9,
                           "frac_of_measured_hbm": bytes_layer / t * 1e-9 / hbm_peak}
    # The fused producer (RMSNorm + rotary embedding + paged write) on the same two sizes: per row it reads
    # 1,152 B of kv_a, 256 B of cos/sin and 4 B of slot and writes 1,152 B (gamma stays in cache).
    gamma = torch.ones(LATENT, dtype=torch.bfloat16, device="cuda")
    trig = torch.empty((2, total, 64), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(trig, SEED, 8)
    fused_src = torch.empty((2, total, ROW), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(fused_src, SEED, 3)
    for name, n_rows, slots_for, iters in (("append_fused", rows, lambda i: slot_sets[i % 4], 86),
                                           ("append_fused_layer", total, lambda i: full_slots, 43)):
        def do_fused(i, n_rows=n_rows, slots_for=slots_for):
            b200kv.append_fused(wl.views[i % LAYERS], fused_src[i % 2][:n_rows], gamma, trig[0][:n_rows], trig[1][:n_rows],
                                slots_for(i), status=wl.status)
        t = timeit(do_fused, iters)
        nbytes = n_rows * (ROW * 2 * 2 + 2 * 64 * 2 + 4)
        res[name] = {"rows_per_launch": n_rows, "algorithmic_bytes": nbytes, "us_per_launch": t * 1e6,
                     "achieved_gbs": nbytes / t * 1e-9, "frac_of_measured_hbm": nbytes / t * 1e-9 / hbm_peak}
    # MX quantisation of attention outputs: the decode step's [32, 64 x 512] (latency) and 4,096 such rows.
    for name, n_rows, iters in (("mx_quant_decode_step", BATCH, 86), ("mx_quant_4096_rows", 4096, 20)):
        cols = HEADS * LATENT
        xq = torch.empty((2, n_rows, cols), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(xq, SEED, 9, 0, 1.0 / 64.0)
        q8 = torch.empty((2, n_rows, cols), dtype=torch.uint8, device="cuda")
        sc = torch.empty((2, n_rows, cols // 32), dtype=torch.uint8, device="cuda")
        t = timeit(lambda i: b200kv.mx_quant_e4m3(xq[i % 2], q8[i % 2], sc[i % 2]), iters)
        nbytes = n_rows * cols * 3 + n_rows * cols // 32
        res[name] = {"rows_per_launch": n_rows, "algorithmic_bytes": nbytes, "us_per_launch": t * 1e6,
                     "achieved_gbs": nbytes / t * 1e-9, "frac_of_measured_hbm": nbytes / t * 1e-9 / hbm_peak}
        del xq, q8, sc
    # The sparse-selection indexer on the step's shape: 32 sequences x 4,096 tokens of FP8 index keys (128 wide),
    # 64 index heads, top 512. First version on CUDA cores: its bound is the fp32 arithmetic
    # (32 x 4,096 x 64 x 128 fused multiply-adds), reported as time, with the key bytes it reads for scale.
    n_rows = wl.blocks * BLOCK
    key8 = torch.randint(0, 0x50, (2, n_rows, 128), dtype=torch.uint8, device="cuda")
    q8 = torch.randint(0, 0x50, (BATCH, HEADS, 128), dtype=torch.uint8, device="cuda")
    k_scale = torch.rand((2, n_rows), dtype=torch.float32, device="cuda") * 0.1 + 0.01
    q_scale = torch.rand((BATCH, HEADS), dtype=torch.float32, device="cuda") * 0.1 + 0.01
    w_idx = torch.randn((BATCH, HEADS), dtype=torch.float32, device="cuda").to(torch.bfloat16)
    # (the binding allocates its outputs and workspace per call: inside a captured graph those come from
    # the graph's private pool, so the replay measures the two kernels)
    t = timeit(lambda i: b200kv.indexer_topk(q8, q_scale, w_idx, key8[i % 2], k_scale[i % 2], wl.table, wl.kv_len,
                                             BLOCK, CONTEXT, 512, status=wl.status), 20)
    res["indexer_topk"] = {"sequences": BATCH, "tokens_per_sequence": CONTEXT, "index_heads": HEADS, "k": 512,
                           "us_per_launch": t * 1e6, "key_bytes": n_rows * 132,
                           "gflop": 2.0 * BATCH * CONTEXT * HEADS * 128 * 1e-9,
                           "tflops_fp32": 2.0 * BATCH * CONTEXT * HEADS * 128 / t * 1e-12}
    del src, out_l, out_r, trig, fused_src, key8, k_scale
    return res


def run_b200_arm(args):
    import torch
    import torch.distributed as dist

    import b200kv

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    variant = {"auto": b200kv.DECODE_AUTO, "simt": b200kv.DECODE_SIMT, "tcgen05": b200kv.DECODE_TCGEN05}[args.variant]
    hbm_peak, tflops_peak, peak_kind = measured_peaks()

    wl = Workload(torch, b200kv, seed_offset=rank)
    err = check_against_oracle(torch, b200kv, wl, variant)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def attention_only():
        for layer in range(LAYERS):
            wl.kv.mla_decode(wl.q[layer], wl.views[layer], wl.table, wl.kv_len, BLOCK, SCALE, out=wl.out[layer],
                             workspace=wl.ws, variant=variant, status=wl.status, stable_tables=True)

    # The 43-layer step is launch-bound from Python (about 15 us of interpreter time per C-ABI call), so the
    # step is captured once in a CUDA graph and replayed: the timed region holds kernels only.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    fused = args.variant != "simt" and not args.separate_append
    if fused:
        # The fused append must leave the pool as the append kernel does: one layer, bit for bit.
        wl.pool[0].index_fill_(0, wl.slots.long(), 0)
        new0 = wl.new_rows[0]
        b200kv.mla_decode(wl.q[0], wl.views[0], wl.table, wl.kv_len, BLOCK, SCALE, out=wl.out[0], workspace=wl.ws,
                          variant=variant, status=wl.status, new_rows=(new0[:, :LATENT], new0[:, LATENT:]))
        torch.cuda.synchronize()
        if not torch.equal(wl.pool[0][wl.slots.long()].view(torch.int16), new0.view(torch.int16)):
            raise RuntimeError("fused append: the pool rows differ from the appended rows")
    with torch.cuda.stream(side):
        wl.step_resident(variant, fused=fused)
        attention_only()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    class Eager:
        def __init__(self, fn):
            self.fn = fn

        def replay(self):
            self.fn()

    if args.no_graph:
        g_step, g_attn = Eager(lambda: wl.step_resident(variant, fused=fused)), Eager(attention_only)
    else:
        g_step = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_step):
            wl.step_resident(variant, fused=fused)
        g_attn = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_attn):
            attention_only()
    launches_per_step = LAYERS * (2 if fused else 3)  # (append,) decode, finalize/merge per layer

    # ---- device-resident timing (value) ----
    for _ in range(args.warmup):
        g_step.replay()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        g_step.replay()
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    # the dominant kernel alone: 43 attention launches (one per layer pool) per replay
    a0 = torch.cuda.Event(enable_timing=True)
    a1 = torch.cuda.Event(enable_timing=True)
    g_attn.replay()
    a0.record()
    for _ in range(args.steps):
        g_attn.replay()
    a1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    attn_ms = a0.elapsed_time(a1) / (args.steps * LAYERS)
    st = wl.status.cpu().tolist()
    if st[0] != 0:
        raise RuntimeError(f"device status word reports {st}")

    def measure_e2e():
        # ---- end-to-end timing through the C ABI with host buffers (e2e) ----
        h_q = torch.empty((LAYERS, BATCH, HEADS, ROW), dtype=torch.bfloat16).pin_memory()
        h_new = torch.empty((LAYERS, BATCH, ROW), dtype=torch.bfloat16).pin_memory()
        h_slots = torch.from_numpy(wl.slots_np).pin_memory()
        h_out = torch.empty((LAYERS, BATCH, HEADS, LATENT), dtype=torch.bfloat16).pin_memory()
        h_q.copy_(wl.q.cpu())
        h_new.copy_(wl.new_rows.cpu())
        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        d_q = [torch.empty_like(wl.q[0]) for _ in range(2)]
        d_new = [torch.empty_like(wl.new_rows[0]) for _ in range(2)]
        d_out = [torch.empty_like(wl.out[0]) for _ in range(2)]
        d_slots = torch.empty_like(wl.slots)

        def step_e2e():
            # Layer l's inputs are uploaded on one stream while layer l-1 computes and layer l-2's result is
            # read back on a third; two buffers per direction. Every byte the step consumes starts in pinned
            # host memory and every result ends there.
            compute = torch.cuda.current_stream()
            in_ready = [None, None]
            in_free = [None, None]
            out_ready = [None, None]
            out_free = [None, None]
            copy_in.wait_stream(compute)
            copy_out.wait_stream(compute)
            with torch.cuda.stream(copy_in):
                d_slots.copy_(h_slots, non_blocking=True)
            for layer in range(LAYERS):
                s = layer & 1
                with torch.cuda.stream(copy_in):
                    if in_free[s] is not None:
                        copy_in.wait_event(in_free[s])
                    d_q[s].copy_(h_q[layer], non_blocking=True)
                    d_new[s].copy_(h_new[layer], non_blocking=True)
                    in_ready[s] = torch.cuda.Event()
                    in_ready[s].record(copy_in)
                compute.wait_event(in_ready[s])
                if out_free[s] is not None:
                    compute.wait_event(out_free[s])
                if not fused:
                    wl.kv.append(wl.views[layer], d_new[s][:, :LATENT], d_new[s][:, LATENT:], d_slots, status=wl.status)
                wl.kv.mla_decode(d_q[s], wl.views[layer], wl.table, wl.kv_len, BLOCK, SCALE, out=d_out[s],
                                 workspace=wl.ws, variant=variant, status=wl.status,
                                 new_rows=(d_new[s][:, :LATENT], d_new[s][:, LATENT:]) if fused else None,
                                 stable_tables=True)
                in_free[s] = torch.cuda.Event()
                in_free[s].record(compute)
                out_ready[s] = torch.cuda.Event()
                out_ready[s].record(compute)
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(out_ready[s])
                    h_out[layer].copy_(d_out[s], non_blocking=True)
                    out_free[s] = torch.cuda.Event()
                    out_free[s].record(copy_out)
            compute.wait_stream(copy_in)
            compute.wait_stream(copy_out)

        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_e2e()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g_e2e = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_e2e):
            step_e2e()
        for _ in range(max(1, args.warmup // 2)):
            g_e2e.replay()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            g_e2e.replay()
        e1.record()
        barrier()
        e2e_ms_total = e0.elapsed_time(e1)
        # the read-back result is the device result, bit for bit
        if not torch.equal(h_out[LAYERS - 1].view(torch.int16), wl.out[LAYERS - 1].cpu().view(torch.int16)):
            raise RuntimeError("bench self-check failed: end-to-end output differs from the resident run")
        return e2e_ms_total

    e2e_ms_total = float('nan') if args.skip_e2e else measure_e2e()
    h2d = LAYERS * (BATCH * HEADS * ROW * 2 + BATCH * ROW * 2) + BATCH * 4
    d2h = LAYERS * BATCH * HEADS * LATENT * 2

    times = torch.tensor([ms_total, e2e_ms_total, attn_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms_total, attn_ms = (float(x) for x in times.cpu())

    move = (measure_move_kernels(torch, b200kv, wl, hbm_peak, use_graph=not args.no_graph)
            if (rank == 0 and not args.skip_move) else None)
    if rank == 0:
        cpu_value, cpu_sample_desc, cpu_threads = (cpu_sample() if (world == 1 and not args.skip_cpu)
                                                    else (None, "skipped (rank 0 at N=1 only)", 0))
        ms_per_step = ms_total / args.steps
        value = world * BATCH / (ms_per_step * 1e-3)
        achieved = ATTN_BYTES_PER_LAUNCH / (attn_ms * 1e-3) * 1e-9
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[1]: B=32 x ctx 4096 per GPU, 43 layers, block 64, seeded permuted "
                                   "block tables, latent KV ~ N(0,1) bf16, 64 heads x 576",
                       "l2": "inputs larger than L2 (151 MB per layer, 6.49 GB pool walked layer by layer)",
                       "launch": "one CUDA graph replay per step (43 x decode with the append fused in + finalize)"
                                 if fused else "one CUDA graph replay per step (43 x append + decode + finalize)",
                       "decode_variant": args.variant, "self_check_max_abs_err": err,
                       "parallelism": f"sequence-partitioned x{world} (no collective)"},
            "roofline": {"kernel": "MlaDecodeTcKernel + MlaFinalizeKernel" if args.variant != "simt"
                         else "MlaDecodeSimtKernel + LseMergeKernel",
                         "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_kind": peak_kind,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH if args.variant != "simt" else None,
                         "traffic_source": "ncu capture of MlaDecodeTcKernel at this workload's shape "
                                           "(profiles/mla_decode_tc_b32x4k_2layers.md): DRAM read 153.83 MB "
                                           "+ write 4.91 MB per launch",
                         "algorithmic_bytes_per_launch": ATTN_BYTES_PER_LAUNCH, "us_per_launch": attn_ms * 1e3,
                         "tflops": ATTN_FLOPS_PER_LAUNCH / (attn_ms * 1e-3) * 1e-12,
                         "frac_of_measured_bf16_peak": ATTN_FLOPS_PER_LAUNCH / (attn_ms * 1e-3) * 1e-12 / tflops_peak},
            "move_kernels": move,
            "cpu_baseline": {"value": cpu_value, "unit": "tokens/s", "cores": cpu_threads, "kind": "port",
                             "sample": cpu_sample_desc},
            "e2e": {"value": None if args.skip_e2e else world * BATCH / (e2e_ms_total / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": None if args.skip_e2e else e2e_ms_total / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------
# The two multi-GPU configurations (not the driver's default workload; run with --workload)
# ---------------------------------------------------------------------------------------------------
def run_extra_workload(args):
    """--workload ragged : configs[2], 256 ragged sequences partitioned over the ranks by length
                           (no collective), fragmented tables, 16 decode steps per timed run.
       --workload longctx: configs[3], one 262,144-token sequence split by KV range over the ranks; every
                           layer ends with an all-gather of the partials (NCCL) and the LSE merge."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import b200kv
    import kvo
    import scenarios
    from b200kv import dist as kvdist

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    hbm_peak, _, peak_kind = measured_peaks()
    layers = args.layers
    status = b200kv.new_status()

    if args.workload == "ragged":
        lens_all = scenarios.ragged_lengths(256, 512, 32768)
        ranks, loads = kvdist.partition_sequences(lens_all, world)
        kv_len_np = lens_all[ranks == rank].astype(np.int32)
        nseq = len(kv_len_np)
        blocks = int(sum(scenarios.blocks_for(int(n) + 16, BLOCK) for n in kv_len_np)) + 8
        table_np = scenarios.fragmented_tables(kv_len_np + 16, BLOCK, blocks)
        pool = torch.empty((layers, blocks * BLOCK, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(pool, SEED + rank, kvo.STREAM_KV)
        q = torch.empty((nseq, HEADS, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(q, SEED + rank, kvo.STREAM_Q, 0, SCALE)
        new = torch.empty((nseq, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(new, SEED + rank, kvo.STREAM_NEW)
        out = torch.empty((nseq, HEADS, LATENT), dtype=torch.bfloat16, device="cuda")
        table = torch.from_numpy(table_np).cuda()
        views = [b200kv.pool_view(pool[l]) for l in range(layers)]
        ws = torch.empty(b200kv.decode_workspace_bytes(nseq), dtype=torch.uint8, device="cuda")
        decode_steps = 16
        # lengths and slots of each of the 16 consecutive decode steps, precomputed on the device
        lens_steps = [torch.from_numpy(kv_len_np + i + 1).cuda() for i in range(decode_steps)]
        slots_steps = []
        for i in range(decode_steps):
            pos = kv_len_np.astype(np.int64) + i
            slots_steps.append(torch.from_numpy(
                (table_np[np.arange(nseq), pos // BLOCK].astype(np.int64) * BLOCK + pos % BLOCK).astype(np.int32)).cuda())

        def step():
            for i in range(decode_steps):
                for l in range(layers):
                    b200kv.append(views[l], new[:, :LATENT], new[:, LATENT:], slots_steps[i], status=status)
                    b200kv.mla_decode(q, views[l], table, lens_steps[i], BLOCK, SCALE, out=out, workspace=ws,
                                      status=status)
        tokens_per_step = 256 * decode_steps
        bytes_per_step = float(sum(int((kv_len_np + i + 1).sum()) for i in range(decode_steps))) * ROW * 2 * layers
        desc = (f"configs[2]: 256 sequences, lengths 512..32768 (seeded), LPT partition over {world} rank(s) "
                f"(rank 0 holds {nseq} sequences, load imbalance {loads.max() / loads.mean():.4f}), fragmented tables, "
                f"{decode_steps} decode steps per run, {layers} of 43 layers resident")
    else:
        n = 262144
        begin, length = kvdist.split_kv_range(n, BLOCK, world, rank)
        my_blocks = scenarios.blocks_for(length, BLOCK)
        total_blocks = n // BLOCK
        # this rank's pool holds only its block range; its table column j maps block begin/BLOCK + j
        table_np = np.zeros((1, total_blocks), dtype=np.int32)
        table_np[0, begin // BLOCK: begin // BLOCK + my_blocks] = kvo.permutation(my_blocks, seed=SEED + rank)
        pool = torch.empty((layers, my_blocks * BLOCK, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(pool, SEED + rank, kvo.STREAM_KV)
        q = torch.empty((1, HEADS, ROW), dtype=torch.bfloat16, device="cuda")
        b200kv.fill_normal_bf16(q, SEED, kvo.STREAM_Q, 0, SCALE)
        table = torch.from_numpy(table_np).cuda()
        lens = torch.tensor([length], dtype=torch.int32, device="cuda")
        begins = torch.tensor([begin], dtype=torch.int32, device="cuda")
        views = [b200kv.pool_view(pool[l]) for l in range(layers)]
        ws = torch.empty(b200kv.decode_workspace_bytes(1), dtype=torch.uint8, device="cuda")
        po = torch.empty((HEADS, LATENT), dtype=torch.float32, device="cuda")
        pm = torch.empty((HEADS,), dtype=torch.float32, device="cuda")
        pl = torch.empty((HEADS,), dtype=torch.float32, device="cuda")
        out = torch.empty((HEADS, LATENT), dtype=torch.bfloat16, device="cuda")
        lse = torch.empty((HEADS,), dtype=torch.float32, device="cuda")

        exchange = kvdist.PeerExchange(HEADS) if args.exchange == "peer" else None

        def step():
            for l in range(layers):
                b200kv.mla_decode(q, views[l], table, lens, BLOCK, SCALE, kv_begin=begins,
                                  partial=(po.view(1, HEADS, LATENT), pm.view(1, HEADS), pl.view(1, HEADS)),
                                  workspace=ws, status=status)
                if exchange is not None:
                    exchange.merge(po, pm, pl, out, lse, status=status)
                elif world > 1:
                    kvdist.merge_across_ranks(po, pm, pl, out, lse)
                else:
                    b200kv.lse_merge(po.view(1, HEADS, LATENT), pm.view(1, HEADS), pl.view(1, HEADS), out, lse)
        tokens_per_step = 1
        bytes_per_step = float(length) * ROW * 2 * layers  # this rank's shard: the roofline is per GPU
        how = ("partials pushed into every rank's inbox over peer memory (NVLink), merged by a kernel that waits for "
               "the peers' flags" if exchange is not None else "all-gather of 131,584-byte partials (NCCL) + LSE merge")
        desc = (f"configs[3]: one sequence of {n} tokens split by KV range over {world} rank(s) "
                f"({length} tokens on rank 0), per layer: {how}; {layers} of 43 layers")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, args.warmup)):
        step()
    barrier()
    run_step = step
    use_graph = not args.no_graph and not (args.workload == "longctx" and args.exchange == "nccl" and world > 1)
    if use_graph:
        # One CUDA graph per step (a C-ABI call from Python costs more host time than these kernels run).
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run_step = graph.replay
        for _ in range(3):
            run_step()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    st = status.cpu().tolist()
    if st[0] != 0:
        raise RuntimeError(f"device status word reports {st}")
    if rank == 0:
        scale43 = 43.0 / layers
        gbs = bytes_per_step / (ms * 1e-3) * 1e-9
        print(json.dumps({
            "metric": f"decode tokens/s ({args.workload})", "value": tokens_per_step / (ms * scale43 * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms * scale43, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": desc},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                         "frac": gbs / hbm_peak, "peak_kind": peak_kind,
                         "note": "rank 0's KV bytes per step over the step time, launch overhead included"},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--variant", default="auto", choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--layers", type=int, default=43, help="fewer layers give a small case for profiler captures")
    ap.add_argument("--no-graph", action="store_true", help="launch step by step instead of replaying CUDA graphs")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-move", action="store_true")
    ap.add_argument("--separate-append", action="store_true",
                    help="append as a launch of its own before each attention launch (default: fused into it)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="longctx only: merge the shards over peer memory (default) or with an NCCL all-gather")
    ap.add_argument("--workload", default="batched", choices=["batched", "ragged", "longctx"],
                    help="batched = configs[1] (the driver's workload); ragged / longctx = the multi-GPU configurations")
    args = ap.parse_args()
    global LAYERS
    LAYERS = args.layers
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload != "batched":
        run_extra_workload(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
