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

WORKLOAD_TEXT = ("configs[1]: B=32 x ctx 4096 per GPU, 43 layers, block 64, seeded permuted block tables, "
                 "latent KV ~ N(0,1) bf16, 64 heads x 576")
HBM_SPEC_GBS = 8000.0   # the nominal figure the goal is stated against; fractions are reported against both

ATTN_BYTES_PER_LAUNCH = BATCH * CONTEXT * ROW * 2 + BATCH * HEADS * ROW * 2 + BATCH * HEADS * LATENT * 2
# DRAM bytes of the decode kernel of one attention launch from the committed ncu capture of the 2-layer case
# (dram__bytes_read.sum + dram__bytes_write.sum, profiles/mla_decode_tc_b32x4k_2layers.md; the merge kernel
# reads the partials from L2 in a warm run). An annotation: the achieved figure is computed from the algorithmic
# bytes above.
NCU_DRAM_BYTES_PER_LAUNCH = 153_440_000 + 4_350_000
ATTN_FLOPS_PER_LAUNCH = BATCH * CONTEXT * HEADS * (ROW + LATENT) * 2


def host_threads() -> int:
    """Host threads this process may use (torchrun exports OMP_NUM_THREADS=1, which is not the machine)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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
# CPU reference arm: the oracle port (the reference's own operators for this path are closed binaries)
# ---------------------------------------------------------------------------------------------------
class CpuSampler:
    """Times the oracle's append + attention on a bounded sample of the step: `layers` layers x `seqs`
    sequences at the full 4096-token context, all host threads, scaled linearly to the full step."""

    def __init__(self):
        import numpy as np

        import kvo

        self.np, self.kvo = np, kvo
        kvo.lib().kvo_set_num_threads(host_threads())  # every host thread, whatever the launcher exported
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
        "config": {"workload": WORKLOAD_TEXT,
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
    """Device-resident state of configs[1] on one GPU. Every buffer the path touches is carved from ONE device
    allocation by the library's static arena, in the engine's order: reserve the KV spans (two layer-major caches,
    block table, slots, lengths) and the step's activations, note the workspace, commit, seal; a layer's pool is
    base + layer * bytes (b200kv_kv_cache_layer_view). torch only wraps the addresses."""

    def __init__(self, torch, b200kv, seed_offset: int = 0):
        import numpy as np

        import kvo

        self.torch, self.kv = torch, b200kv
        blocks_per_seq = CONTEXT // BLOCK
        self.blocks = BATCH * blocks_per_seq
        rows = self.blocks * BLOCK
        arena = b200kv.Arena(b200kv.ARENA_DEVICE)
        cache = arena.reserve_kv_cache_batched(self.blocks, BLOCK, LAYERS, BATCH, blocks_per_seq, BATCH)
        h_q = arena.reserve("attn.q", LAYERS * BATCH * HEADS * ROW * 2)
        h_new = arena.reserve("attn.new_rows", LAYERS * BATCH * ROW * 2)
        h_out = arena.reserve("attn.out", LAYERS * BATCH * HEADS * LATENT * 2)
        h_status = arena.reserve("attn.status", 16)
        arena.note_workspace(b200kv.decode_workspace_bytes(BATCH, HEADS))
        arena.commit()
        arena.commit_workspace()
        arena.seal()
        if arena.allocations != 2:
            raise RuntimeError(f"the arena made {arena.allocations} allocations (one for the spans, one workspace expected)")
        self.arena, self.cache = arena, cache
        bf16, i32 = torch.bfloat16, torch.int32
        self.latent = arena.tensor(cache.latent_handle, (LAYERS, rows, LATENT), bf16)
        self.rope = arena.tensor(cache.rope_handle, (LAYERS, rows, ROW - LATENT), bf16)
        self.table = arena.tensor(cache.block_table_handle, (BATCH, blocks_per_seq), i32)
        self.slots = arena.tensor(cache.slot_mapping_handle, (BATCH,), i32)
        self.kv_len = arena.tensor(cache.seq_lens_handle, (BATCH,), i32)
        self.q = arena.tensor(h_q, (LAYERS, BATCH, HEADS, ROW), bf16)
        self.new_rows = arena.tensor(h_new, (LAYERS, BATCH, ROW), bf16)
        self.out = arena.tensor(h_out, (LAYERS, BATCH, HEADS, LATENT), bf16)
        self.status = arena.tensor(h_status, (4,), i32)
        self.ws = b200kv.device_tensor(arena.workspace, (arena.workspace_bytes,), torch.uint8)
        b200kv.fill_normal_bf16(self.latent, SEED + seed_offset, kvo.STREAM_KV)
        b200kv.fill_normal_bf16(self.rope, SEED + seed_offset, kvo.STREAM_KV + 64)
        table = kvo.permutation(self.blocks, seed=SEED + seed_offset).reshape(BATCH, blocks_per_seq)
        self.table_np = table
        self.table.copy_(torch.from_numpy(table).cuda())
        self.kv_len.fill_(CONTEXT)
        slots = (table[:, -1].astype(np.int64) * BLOCK + (CONTEXT - 1) % BLOCK).astype(np.int32)
        self.slots_np = slots
        self.slots.copy_(torch.from_numpy(slots).cuda())
        b200kv.fill_normal_bf16(self.q, SEED + seed_offset, kvo.STREAM_Q, 0, SCALE)
        b200kv.fill_normal_bf16(self.new_rows, SEED + seed_offset, kvo.STREAM_NEW)
        self.views = [arena.layer_view(cache, layer) for layer in range(LAYERS)]
        self.launches = 0

    def close(self):
        self.torch.cuda.synchronize()
        for name in ("latent", "rope", "table", "slots", "kv_len", "q", "new_rows", "out", "status", "ws"):
            setattr(self, name, None)
        self.arena.close()

    def step_resident(self, variant, fused=False):
        """43 layers of append + attention. fused: the append rides in the attention launch (the decode kernel
        writes each sequence's new row before it reads that tile) instead of a launch of its own."""
        for layer in range(LAYERS):
            new = self.new_rows[layer]
            if not fused:
                self.kv.append(self.views[layer], new[:, :LATENT], new[:, LATENT:], self.slots, status=self.status)
            self.kv.mla_decode(self.q[layer], self.views[layer], self.table, self.kv_len, BLOCK, SCALE,
                               out=self.out[layer], workspace=self.ws, variant=variant, status=self.status,
                               new_rows=(new[:, :LATENT], new[:, LATENT:]) if fused else None,
                               stable_tables=True)  # table and lengths are uploaded before the step
            self.launches += 2 if fused else 3


def check_against_oracle(torch, b200kv, wl: Workload, variant) -> float:
    """Two sequences of one layer, copied back and recomputed by the oracle (the GPU tests hold all 32)."""
    import numpy as np

    import kvo

    layer = min(7, LAYERS - 1)
    wl.step_resident(variant)
    torch.cuda.synchronize()
    worst = 0.0
    for b in (5, 31):
        rows = (wl.table_np[b].astype(np.int64)[:, None] * BLOCK + np.arange(BLOCK)[None, :]).reshape(-1)
        idx = torch.from_numpy(rows).cuda()
        kv_rows = torch.cat([wl.latent[layer][idx], wl.rope[layer][idx]], dim=1).contiguous()
        pool_np = kv_rows.view(torch.int16).cpu().numpy().view(np.uint16)
        q_np = wl.q[layer, b].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)[None]
        table = np.arange(CONTEXT // BLOCK, dtype=np.int32)[None]
        want, _ = kvo.mla_decode(q_np, pool_np, table, np.array([CONTEXT], np.int32), BLOCK, SCALE, use_double=True)
        got = wl.out[layer, b].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        err = float(np.abs(kvo.bf16_to_f32(got) - kvo.bf16_to_f32(want[0])).max())
        if not err <= 2e-3:
            raise RuntimeError(f"bench self-check failed: attention differs from the oracle by {err:.3e}")
        worst = max(worst, err)
        # the appended row is in the pool, bit for bit
        slot = int(wl.slots_np[b])
        got_row = torch.cat([wl.latent[layer, slot], wl.rope[layer, slot]])
        if not torch.equal(got_row.view(torch.int16), wl.new_rows[layer, b].view(torch.int16)):
            raise RuntimeError("bench self-check failed: appended row not found in the pool")
    return worst


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
    # The same 16,384 rows as the churn configuration's prefill chunk really presents them: 64 sequences x 256
    # tokens from activations [T][512] and [T][64] into 64-row blocks (runs of 64 consecutive slots) of the two
    # caches.
    lat_src = torch.empty((4, rows, LATENT), dtype=torch.bfloat16, device="cuda")
    rope_src = torch.empty((4, rows, ROW - LATENT), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(lat_src, SEED, 4)
    b200kv.fill_normal_bf16(rope_src, SEED, 5)
    block_ids = torch.randperm(wl.blocks, device="cuda", dtype=torch.int64)
    run_sets = []
    for i in range(4):
        ids = block_ids[i * (rows // BLOCK):(i + 1) * (rows // BLOCK)]
        run_sets.append((ids[:, None] * BLOCK + torch.arange(BLOCK, device="cuda")[None, :]).reshape(-1).to(torch.int32).contiguous())

    def do_append_chunk(i):
        b200kv.append(wl.views[i % LAYERS], lat_src[i % 4], rope_src[i % 4], run_sets[i % 4], status=wl.status)
    t = timeit(do_append_chunk, 86)
    res["append_prefill_chunk"] = {"rows_per_launch": rows, "algorithmic_bytes": bytes_append, "us_per_launch": t * 1e6,
                                   "achieved_gbs": bytes_append / t * 1e-9,
                                   "frac_of_measured_hbm": bytes_append / t * 1e-9 / hbm_peak,
                                   "shape": "64 sequences x 256 tokens into 64-row blocks, sources [T][512] and [T][64]"}
    # What a plain device-to-device copy of the same bytes reaches at this size (one launch of 18.9 MB read and
    # 18.9 MB written, eight source and eight destination buffers in turn so that neither side stays in L2): the
    # ceiling a launch of this size has, whatever the kernel.
    flat_src = torch.empty((8, bytes_append // 4), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(flat_src, SEED, 6)
    flat_dst = torch.empty_like(flat_src)
    t = timeit(lambda i: flat_dst[i % 8].copy_(flat_src[(i + 3) % 8]), 88)
    res["plain_copy_same_bytes"] = {"bytes": bytes_append, "us_per_launch": t * 1e6,
                                    "achieved_gbs": bytes_append / t * 1e-9,
                                    "frac_of_measured_hbm": bytes_append / t * 1e-9 / hbm_peak}
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
    # The sparse path on the step's shape: the indexer over 32 sequences x 4,096 tokens of FP8 index keys (128
    # wide, 64 index heads, top 512), then attention over the 512 selected rows of each sequence. The score kernel
    # reads 132 bytes per token (key + key scale) and writes 4; tensor-core variant (FP8 tcgen05) and the exact
    # CUDA-core one. The attention gathers 32 x 512 rows of 1,152 bytes with 16-byte asynchronous copies.
    n_rows = wl.blocks * BLOCK
    key8 = torch.randint(0, 0x50, (8, n_rows, 128), dtype=torch.uint8, device="cuda")  # 8 x 17 MB: larger than L2
    q8 = torch.randint(0, 0x50, (BATCH, HEADS, 128), dtype=torch.uint8, device="cuda")
    k_scale = torch.rand((8, n_rows), dtype=torch.float32, device="cuda") * 0.1 + 0.01
    q_scale = torch.rand((BATCH, HEADS), dtype=torch.float32, device="cuda") * 0.1 + 0.01
    w_idx = torch.randn((BATCH, HEADS), dtype=torch.float32, device="cuda").to(torch.bfloat16)
    # (the binding allocates its outputs and workspace per call: inside a captured graph those come from
    # the graph's private pool, so the replay measures the two kernels)
    idx_bytes = BATCH * CONTEXT * (128 + 4 + 4)
    for name, variant in (("indexer_topk", b200kv.INDEXER_TCGEN05), ("indexer_topk_exact", b200kv.INDEXER_EXACT)):
        t = timeit(lambda i: b200kv.indexer_topk(q8, q_scale, w_idx, key8[i % 8], k_scale[i % 8], wl.table, wl.kv_len,
                                                 BLOCK, CONTEXT, 512, status=wl.status, variant=variant), 24)
        res[name] = {"sequences": BATCH, "tokens_per_sequence": CONTEXT, "index_heads": HEADS, "k": 512,
                     "kernels": "score (FP8 tcgen05) + radix select" if variant == b200kv.INDEXER_TCGEN05
                                else "score (fp32 chains on CUDA cores) + radix select",
                     "us_per_launch": t * 1e6, "score_bytes": idx_bytes,
                     "gflop": 2.0 * BATCH * CONTEXT * HEADS * 128 * 1e-9,
                     "tflops": 2.0 * BATCH * CONTEXT * HEADS * 128 / t * 1e-12}
    index, n_sel = b200kv.indexer_topk(q8, q_scale, w_idx, key8[0], k_scale[0], wl.table, wl.kv_len, BLOCK, CONTEXT, 512,
                                       status=wl.status)
    rows_sel = b200kv.resolve_rows(wl.table, BLOCK, index, n_sel, wl.blocks * BLOCK, status=wl.status)
    for name, variant in (("sparse_decode_512", b200kv.DECODE_TCGEN05), ("sparse_decode_512_simt", b200kv.DECODE_SIMT)):
        t = timeit(lambda i: b200kv.mla_decode(wl.q[i % LAYERS], wl.views[i % LAYERS], None, n_sel, BLOCK, SCALE,
                                               out=wl.out[i % LAYERS], workspace=wl.ws, variant=variant, status=wl.status,
                                               row_index=rows_sel), 43)
        sel_bytes = BATCH * 512 * ROW * 2 + BATCH * HEADS * (ROW + LATENT) * 2
        res[name] = {"sequences": BATCH, "rows_per_sequence": 512, "algorithmic_bytes": sel_bytes,
                     "kernel": "MlaDecodeTcKernel<gathered> (cp.async rows, swizzled) + MlaFinalizeKernel"
                               if variant == b200kv.DECODE_TCGEN05 else "MlaDecodeSimtKernel over single-row blocks",
                     "us_per_launch": t * 1e6, "achieved_gbs": sel_bytes / t * 1e-9,
                     "frac_of_measured_hbm": sel_bytes / t * 1e-9 / hbm_peak}
    # The sparse step as the model would run it per layer: indexer (scores, selection, pool rows) then the gathered
    # decode, two calls and four kernels.
    rows_buf = torch.empty((BATCH, 512), dtype=torch.int32, device="cuda")

    def sparse_layer(i):
        layer = i % LAYERS
        _, n_s = b200kv.indexer_topk(q8, q_scale, w_idx, key8[i % 8], k_scale[i % 8], wl.table, wl.kv_len, BLOCK, CONTEXT, 512,
                                     status=wl.status, rows_out=rows_buf)
        b200kv.mla_decode(wl.q[layer], wl.views[layer], None, n_s, BLOCK, SCALE, out=wl.out[layer], workspace=wl.ws,
                          variant=b200kv.DECODE_TCGEN05, status=wl.status, row_index=rows_buf)

    t = timeit(sparse_layer, 24)
    res["sparse_layer_top512"] = {"what": "indexer (FP8 tcgen05 scores, select, rows) + attention over the 32 x 512 selected rows",
                                  "us_per_layer": t * 1e6}
    del rows_buf
    # Where the selection pays: 8 sequences of 32,768 tokens. Dense attention reads 302 MB a layer; the sparse layer
    # reads 34.6 MB of index keys and 8 x 512 rows.
    b2, ctx2 = 8, 32768
    rows2 = b2 * ctx2
    pool2 = torch.empty((2, rows2, ROW), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(pool2, SEED, 21)
    table2 = torch.randperm(rows2 // BLOCK, device="cuda").to(torch.int32).view(b2, ctx2 // BLOCK).contiguous()
    lens2 = torch.full((b2,), ctx2, dtype=torch.int32, device="cuda")
    key2 = torch.randint(0, 0x50, (2, rows2, 128), dtype=torch.uint8, device="cuda")
    ks2 = torch.rand((2, rows2), dtype=torch.float32, device="cuda") * 0.1 + 0.01
    ws2 = torch.empty(b200kv.decode_workspace_bytes(b2), dtype=torch.uint8, device="cuda")
    out2 = torch.empty((b2, HEADS, LATENT), dtype=torch.bfloat16, device="cuda")
    rows_buf2 = torch.empty((b2, 512), dtype=torch.int32, device="cuda")
    views2 = [b200kv.pool_view(pool2[i]) for i in range(2)]

    def dense_long(i):
        b200kv.mla_decode(wl.q[i % LAYERS][:b2], views2[i % 2], table2, lens2, BLOCK, SCALE, out=out2, workspace=ws2,
                          variant=b200kv.DECODE_TCGEN05, status=wl.status, stable_tables=True)

    def sparse_long(i):
        _, n_s = b200kv.indexer_topk(q8[:b2], q_scale[:b2], w_idx[:b2], key2[i % 2], ks2[i % 2], table2, lens2, BLOCK, ctx2, 512,
                                     status=wl.status, rows_out=rows_buf2)
        b200kv.mla_decode(wl.q[i % LAYERS][:b2], views2[i % 2], None, n_s, BLOCK, SCALE, out=out2, workspace=ws2,
                          variant=b200kv.DECODE_TCGEN05, status=wl.status, row_index=rows_buf2)

    t_dense, t_sparse = timeit(dense_long, 8), timeit(sparse_long, 8)
    res["long_context_8x32k"] = {"dense_attention_us_per_layer": t_dense * 1e6, "sparse_layer_top512_us_per_layer": t_sparse * 1e6,
                                 "dense_bytes": rows2 * ROW * 2, "sparse_bytes": rows2 * 136 + b2 * 512 * ROW * 2}
    del pool2, key2, ks2, ws2, out2, rows_buf2, table2, lens2, views2
    del index, n_sel, rows_sel
    # Attention with its output's MX quantisation (the reference's stage 10 behind stage 9): written by the merge
    # kernel itself against a quantiser launch of its own behind the attention.
    aq8 = torch.empty((BATCH, HEADS, LATENT), dtype=torch.uint8, device="cuda")
    asc = torch.empty((BATCH, HEADS, LATENT // 32), dtype=torch.uint8, device="cuda")

    def attend(i, fused_quant):
        layer = i % LAYERS
        b200kv.mla_decode(wl.q[layer], wl.views[layer], wl.table, wl.kv_len, BLOCK, SCALE, out=wl.out[layer],
                          workspace=wl.ws, variant=b200kv.DECODE_TCGEN05, status=wl.status, stable_tables=True,
                          quantised=(aq8, asc) if fused_quant else None)
        if not fused_quant:
            b200kv.mx_quant_e4m3(wl.out[layer].view(BATCH, HEADS * LATENT), aq8.view(BATCH, -1), asc.view(BATCH, -1))

    for name, fused_quant in (("attention_quant_fused", True), ("attention_then_quant", False)):
        t = timeit(lambda i: attend(i, fused_quant), 43)
        res[name] = {"what": "decode + merge with the MX quantisation as the merge kernel's epilogue" if fused_quant
                             else "decode + merge, then b200kv_mx_quant_e4m3 on the 32 output rows",
                     "us_per_layer": t * 1e6}
    del aq8, asc
    del src, out_l, out_r, trig, fused_src, key8, k_scale, lat_src, rope_src, flat_src, flat_dst
    return res


def capture(torch, fn, warm: int = 1):
    """Runs fn once on a side stream (lazy initialisations), then captures it in a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def timed(torch, run, steps: int, barrier):
    """Milliseconds for `steps` calls of run(), CUDA events on the current stream, a barrier on both sides."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


def measure_e2e(torch, b200kv, wl, variant, fused, args, barrier):
    """The step through the C ABI with HOST buffers: every layer's inputs (q and the new rows, one contiguous
    pinned block and one copy per layer) come up from pinned memory and every layer's output goes back, on
    three streams with four device buffers per direction, captured as one graph. Also measures the same copies
    with no kernels between them: the floor the host link sets for this step at this rank count."""
    n_buf = 4
    in_elems = BATCH * HEADS * ROW + BATCH * ROW
    out_elems = BATCH * HEADS * LATENT
    bf16 = torch.bfloat16
    h_in = torch.empty((LAYERS, in_elems), dtype=bf16).pin_memory()
    h_out = torch.empty((LAYERS, out_elems), dtype=bf16).pin_memory()
    h_slots = torch.from_numpy(wl.slots_np).pin_memory()
    h_in[:, :BATCH * HEADS * ROW].copy_(wl.q.reshape(LAYERS, -1).cpu())
    h_in[:, BATCH * HEADS * ROW:].copy_(wl.new_rows.reshape(LAYERS, -1).cpu())
    d_in = [torch.empty(in_elems, dtype=bf16, device="cuda") for _ in range(n_buf)]
    d_out = [torch.empty((BATCH, HEADS, LATENT), dtype=bf16, device="cuda") for _ in range(n_buf)]
    d_slots = torch.empty_like(wl.slots)
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step(with_kernels: bool):
        compute = torch.cuda.current_stream()
        in_free, out_free = [None] * n_buf, [None] * n_buf
        copy_in.wait_stream(compute)
        copy_out.wait_stream(compute)
        with torch.cuda.stream(copy_in):
            d_slots.copy_(h_slots, non_blocking=True)
        for layer in range(LAYERS):
            s = layer % n_buf
            with torch.cuda.stream(copy_in):
                if in_free[s] is not None:
                    copy_in.wait_event(in_free[s])
                d_in[s].copy_(h_in[layer], non_blocking=True)
                in_ready = torch.cuda.Event()
                in_ready.record(copy_in)
            compute.wait_event(in_ready)
            if out_free[s] is not None:
                compute.wait_event(out_free[s])
            if with_kernels:
                q = d_in[s][:BATCH * HEADS * ROW].view(BATCH, HEADS, ROW)
                new = d_in[s][BATCH * HEADS * ROW:].view(BATCH, ROW)
                if not fused:
                    wl.kv.append(wl.views[layer], new[:, :LATENT], new[:, LATENT:], d_slots, status=wl.status)
                wl.kv.mla_decode(q, wl.views[layer], wl.table, wl.kv_len, BLOCK, SCALE, out=d_out[s], workspace=wl.ws,
                                 variant=variant, status=wl.status,
                                 new_rows=(new[:, :LATENT], new[:, LATENT:]) if fused else None, stable_tables=True)
            in_free[s] = torch.cuda.Event()
            in_free[s].record(compute)
            out_ready = torch.cuda.Event()
            out_ready.record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(out_ready)
                h_out[layer].copy_(d_out[s].view(-1), non_blocking=True)
                out_free[s] = torch.cuda.Event()
                out_free[s].record(copy_out)
        compute.wait_stream(copy_in)
        compute.wait_stream(copy_out)

    g_e2e = capture(torch, lambda: step(True))
    g_floor = capture(torch, lambda: step(False))
    for _ in range(max(3, args.warmup // 2)):
        g_e2e.replay()
    ms_e2e = timed(torch, g_e2e.replay, args.steps, barrier)
    # the read-back result is the device result, bit for bit
    if not torch.equal(h_out[LAYERS - 1].view(torch.int16), wl.out[LAYERS - 1].reshape(-1).cpu().view(torch.int16)):
        raise RuntimeError("bench self-check failed: end-to-end output differs from the resident run")
    for _ in range(3):
        g_floor.replay()
    ms_floor = timed(torch, g_floor.replay, args.steps, barrier)
    return ms_e2e, ms_floor


# ---------------------------------------------------------------------------------------------------
# The two multi-GPU configurations: legs of the default run (a few layers resident) and, with --workload,
# runs of their own
# ---------------------------------------------------------------------------------------------------
def leg_ragged(torch, dist, b200kv, layers: int, steps: int, use_graph: bool = True):
    """configs[2]: 256 ragged sequences (lengths 512..32768 from a seed) partitioned over the ranks by length
    (no data-path collective), fragmented tables, 16 consecutive decode steps per run with the append fused
    into each attention launch. Three of rank 0's sequences are checked against the oracle."""
    import numpy as np

    import kvo
    import scenarios
    from b200kv import dist as kvdist

    rank, world, _ = dist_env()
    hbm_peak, _, peak_kind = measured_peaks()
    status = b200kv.new_status()
    lens_all = scenarios.ragged_lengths(256, 512, 32768)
    ranks, loads = kvdist.partition_sequences(lens_all, world)
    kv_len_np = lens_all[ranks == rank].astype(np.int32)
    nseq = len(kv_len_np)
    decode_steps = 16
    blocks = int(sum(scenarios.blocks_for(int(n) + decode_steps, BLOCK) for n in kv_len_np)) + 8
    table_np = scenarios.fragmented_tables(kv_len_np + decode_steps, BLOCK, blocks)
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
    # lengths of each of the 16 consecutive decode steps (the new token included), precomputed on the device
    lens_steps = [torch.from_numpy(kv_len_np + i + 1).cuda() for i in range(decode_steps)]

    def step():
        for i in range(decode_steps):
            for l in range(layers):
                b200kv.mla_decode(q, views[l], table, lens_steps[i], BLOCK, SCALE, out=out, workspace=ws, status=status,
                                  new_rows=(new[:, :LATENT], new[:, LATENT:]), stable_tables=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    run = capture(torch, step).replay if use_graph else step
    for _ in range(2):
        run()
    ms = timed(torch, run, steps, barrier) / steps
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    st = status.cpu().tolist()
    if st[0] != 0:
        raise RuntimeError(f"ragged leg: device status word reports {st}")
    err = None
    if rank == 0:
        # the last layer's output of the last decode step, three sequences, against the oracle
        final_len = kv_len_np + decode_steps
        err = 0.0
        for b in (0, nseq // 2, nseq - 1):
            n = int(final_len[b])
            tok = np.arange(n)
            rows = table_np[b, tok // BLOCK].astype(np.int64) * BLOCK + tok % BLOCK
            kv_rows = pool[layers - 1][torch.from_numpy(rows).cuda()].contiguous()
            pool_np = kv_rows.view(torch.int16).cpu().numpy().view(np.uint16)
            q_np = q[b].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)[None]
            ident = np.arange(scenarios.blocks_for(n, BLOCK), dtype=np.int32)[None]
            want, _ = kvo.mla_decode(q_np, pool_np, ident, np.array([n], np.int32), BLOCK, SCALE, use_double=True)
            got = out[b].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            err = max(err, float(np.abs(kvo.bf16_to_f32(got) - kvo.bf16_to_f32(want[0])).max()))
        if not err <= 2e-3:
            raise RuntimeError(f"ragged leg: attention differs from the oracle by {err:.3e}")
    scale43 = 43.0 / layers
    tokens = float(sum(int((lens_all + i + 1).sum()) for i in range(decode_steps)))
    my_bytes = float(sum(int((kv_len_np + i + 1).sum()) for i in range(decode_steps))) * ROW * 2 * layers
    gbs = my_bytes / (ms * 1e-3) * 1e-9
    del pool
    return {
        "workload": (f"configs[2]: 256 sequences, lengths 512..32768 (seeded), partitioned over {world} rank(s) by "
                     f"length (rank 0 holds {nseq}, load imbalance {loads.max() / loads.mean():.4f}), fragmented "
                     f"tables, {decode_steps} decode steps per run with the append fused into each launch"),
        "layers_resident": layers, "value": 256 * decode_steps / (ms * scale43 * 1e-3), "unit": "tokens/s",
        "ms_per_run_43_layers": ms * scale43, "context_tokens_per_run": tokens,
        "rank0_hbm_gbs": gbs, "rank0_frac_of_measured_hbm": gbs / hbm_peak, "peak_kind": peak_kind,
        "max_abs_err": err, "scaling": "strong",
    }


def leg_longctx(torch, dist, b200kv, layers: int, steps: int, exchange_kind: str = "peer", use_graph: bool = True,
                max_ctas: int = 0, tokens: int = 262144):
    """configs[3]: one sequence of 262,144 tokens split by KV range over the ranks; every layer ends with the
    exchange of the ranks' partials (peer memory over NVLink, or an NCCL all-gather) and the log-sum-exp merge.
    Rank 0 checks layer 0 against the oracle on 8 heads over the whole sequence."""
    import numpy as np

    import kvo
    import scenarios
    from b200kv import dist as kvdist

    rank, world, _ = dist_env()
    hbm_peak, _, peak_kind = measured_peaks()
    status = b200kv.new_status()
    n = tokens
    begin, length = kvdist.split_kv_range(n, BLOCK, world, rank)
    my_blocks = scenarios.blocks_for(length, BLOCK)
    total_blocks = n // BLOCK
    # this rank's pool holds only its block range; its table column j maps block begin / BLOCK + j
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
    out = torch.empty((layers, HEADS, LATENT), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((HEADS,), dtype=torch.float32, device="cuda")
    exchange = kvdist.PeerExchange(HEADS) if exchange_kind == "peer" else None

    def decode(l):
        b200kv.mla_decode(q, views[l], table, lens, BLOCK, SCALE, kv_begin=begins,
                          partial=(po.view(1, HEADS, LATENT), pm.view(1, HEADS), pl.view(1, HEADS)), workspace=ws,
                          status=status, stable_tables=True, max_ctas=max_ctas)

    def step():
        for l in range(layers):
            if exchange is not None:
                # decode of the shard and the merge across the ranks as one call of two kernels
                exchange.decode_merge(q, views[l], table, lens, BLOCK, SCALE, out[l].view(1, HEADS, LATENT), lse=lse,
                                      kv_begin=begins, workspace=ws, status=status, stable_tables=True,
                                      max_ctas=max_ctas)
                continue
            decode(l)
            if world > 1:
                kvdist.merge_across_ranks(po, pm, pl, out[l], lse)
            else:
                b200kv.lse_merge(po.view(1, HEADS, LATENT), pm.view(1, HEADS), pl.view(1, HEADS), out[l], lse)

    def decode_only():
        for l in range(layers):
            decode(l)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graphs = use_graph and not (exchange is None and world > 1)  # NCCL calls are launched eagerly
    run = capture(torch, step).replay if graphs else step
    run_decode = capture(torch, decode_only).replay if graphs else decode_only
    for _ in range(3):
        run()
    barrier()
    t = torch.tensor([timed(torch, run, steps, barrier) / steps, timed(torch, run_decode, steps, barrier) / steps],
                     dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_decode = (float(x) for x in t.cpu())
    st = status.cpu().tolist()
    if st[0] != 0:
        raise RuntimeError(f"longctx leg: device status word reports {st}")
    err = None
    if rank == 0:
        # Layer 0 of every rank's shard regenerated on the host (the device generator and the oracle's agree bit
        # for bit), the whole sequence attended by the oracle on 8 heads.
        kvo.lib().kvo_set_num_threads(host_threads())
        shards, tables = [], []
        row_base = 0
        for r in range(world):
            _, r_len = kvdist.split_kv_range(n, BLOCK, world, r)
            r_blocks = scenarios.blocks_for(r_len, BLOCK)
            shards.append(kvo.normal_bf16(r_blocks * BLOCK * ROW, kvo.STREAM_KV, seed=SEED + r).reshape(-1, ROW))
            tables.append(kvo.permutation(r_blocks, seed=SEED + r).astype(np.int64) + row_base // BLOCK)
            row_base += r_blocks * BLOCK
        pool_np = np.concatenate(shards)
        table_all = np.concatenate(tables).astype(np.int32)[None]
        heads = np.arange(0, HEADS, 8)
        q_np = q.view(torch.int16).cpu().numpy().view(np.uint16)
        want, _ = kvo.mla_decode(q_np[:, heads], pool_np, table_all, np.array([n], np.int32), BLOCK, SCALE)
        got = out[0].view(torch.int16).cpu().numpy().view(np.uint16)[heads]
        err = float(np.abs(kvo.bf16_to_f32(got) - kvo.bf16_to_f32(want[0])).max())
        if not err <= 2e-3:
            raise RuntimeError(f"longctx leg: attention differs from the oracle by {err:.3e}")
    if exchange is not None:
        barrier()
        exchange.close()
    scale43 = 43.0 / layers
    gbs = float(length) * ROW * 2 * layers / (ms * 1e-3) * 1e-9
    how = ("the kernel that merges the shard's per-CTA partials pushes the result into every rank's inbox over peer "
           "memory (NVLink) and merges what arrives"
           if exchange is not None else "all-gather of 131,584-byte partials (NCCL) + LSE merge")
    del pool
    return {
        "workload": (f"configs[3]: one sequence of {n} tokens split by KV range over {world} rank(s) ({length} tokens "
                     f"on rank 0); per layer: decode of the shard, then {how}"),
        "layers_resident": layers, "ms_per_step_43_layers": ms * scale43, "value": 1.0 / (ms * scale43 * 1e-3),
        "unit": "tokens/s", "us_per_layer": ms * 1e3 / layers, "decode_us_per_layer": ms_decode * 1e3 / layers,
        "exchange_us_per_layer": (ms - ms_decode) * 1e3 / layers, "rank0_hbm_gbs": gbs,
        "rank0_frac_of_measured_hbm": gbs / hbm_peak, "peak_kind": peak_kind, "max_abs_err": err, "scaling": "strong",
    }


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

    fused = args.variant != "simt" and not args.separate_append
    if fused:
        # The fused append must leave the pool as the append kernel does: one layer, bit for bit.
        wl.latent[0].index_fill_(0, wl.slots.long(), 0)
        wl.rope[0].index_fill_(0, wl.slots.long(), 0)
        new0 = wl.new_rows[0]
        b200kv.mla_decode(wl.q[0], wl.views[0], wl.table, wl.kv_len, BLOCK, SCALE, out=wl.out[0], workspace=wl.ws,
                          variant=variant, status=wl.status, new_rows=(new0[:, :LATENT], new0[:, LATENT:]))
        torch.cuda.synchronize()
        got0 = torch.cat([wl.latent[0][wl.slots.long()], wl.rope[0][wl.slots.long()]], dim=1)
        if not torch.equal(got0.view(torch.int16), new0.view(torch.int16)):
            raise RuntimeError("fused append: the pool rows differ from the appended rows")

    # The 43-layer step is launch-bound from Python (about 15 us of interpreter time per C-ABI call), so the
    # step is captured once in a CUDA graph and replayed: the timed region holds kernels only.
    class Eager:
        def __init__(self, fn):
            self.fn = fn

        def replay(self):
            self.fn()

    if args.no_graph:
        wl.step_resident(variant, fused=fused)
        attention_only()
        g_step, g_attn = Eager(lambda: wl.step_resident(variant, fused=fused)), Eager(attention_only)
    else:
        g_step = capture(torch, lambda: wl.step_resident(variant, fused=fused))
        g_attn = capture(torch, attention_only)
    launches_per_step = LAYERS * (2 if fused else 3)  # (append,) decode, finalize/merge per layer

    # ---- device-resident timing (value) ----
    for _ in range(args.warmup):
        g_step.replay()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total = timed(torch, g_step.replay, args.steps, barrier)
    # the dominant kernel alone: 43 attention launches (one per layer pool) per replay
    g_attn.replay()
    attn_ms = timed(torch, g_attn.replay, args.steps, barrier) / (args.steps * LAYERS)
    clocks = sampler.stop() if rank == 0 else None
    st = wl.status.cpu().tolist()
    if st[0] != 0:
        raise RuntimeError(f"device status word reports {st}")

    e2e_ms_total, floor_ms_total = ((float('nan'), float('nan')) if args.skip_e2e
                                    else measure_e2e(torch, b200kv, wl, variant, fused, args, barrier))
    h2d = LAYERS * (BATCH * HEADS * ROW * 2 + BATCH * ROW * 2) + BATCH * 4
    d2h = LAYERS * BATCH * HEADS * LATENT * 2

    times = torch.tensor([ms_total, e2e_ms_total, attn_ms, floor_ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms_total, attn_ms, floor_ms_total = (float(x) for x in times.cpu())

    move = (measure_move_kernels(torch, b200kv, wl, hbm_peak, use_graph=not args.no_graph)
            if (rank == 0 and not args.skip_move) else None)
    wl.close()
    del wl
    torch.cuda.empty_cache()
    # ---- the two multi-GPU configurations, a few layers each, as extra keys of the same line ----
    legs = {}
    if not args.skip_legs:
        legs["longctx"] = leg_longctx(torch, dist, b200kv, layers=min(4, LAYERS), steps=10, use_graph=not args.no_graph)
        torch.cuda.empty_cache()
        legs["ragged"] = leg_ragged(torch, dist, b200kv, layers=min(2, LAYERS), steps=3, use_graph=not args.no_graph)
        torch.cuda.empty_cache()
    if rank == 0:
        cpu_value, cpu_sample_desc, cpu_threads = (cpu_sample() if (world == 1 and not args.skip_cpu)
                                                    else (None, "skipped (rank 0 at N=1 only)", 0))
        ms_per_step = ms_total / args.steps
        value = world * BATCH / (ms_per_step * 1e-3)
        achieved = ATTN_BYTES_PER_LAUNCH / (attn_ms * 1e-3) * 1e-9
        e2e_ms = None if args.skip_e2e else e2e_ms_total / args.steps
        floor_ms = None if args.skip_e2e else floor_ms_total / args.steps
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD_TEXT,
                       "memory": "KV spans, activations and workspace carved from one arena allocation "
                                 "(reserve / commit / seal); per-layer pool = base + layer * bytes",
                       "l2": "inputs larger than L2 (151 MB per layer, 6.49 GB pool walked layer by layer)",
                       "launch": "one CUDA graph replay per step (43 x decode with the append fused in + finalize)"
                                 if fused else "one CUDA graph replay per step (43 x append + decode + finalize)",
                       "decode_variant": args.variant, "self_check_max_abs_err": err,
                       "parallelism": f"sequence-partitioned x{world} (no collective)"},
            "roofline": {"kernel": "MlaDecodeTcKernel + MlaFinalizeKernel" if args.variant != "simt"
                         else "MlaDecodeSimtKernel + LseMergeKernel",
                         "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "peak_kind": peak_kind,
                         "frac_of_8tbs_nominal": achieved / HBM_SPEC_GBS,
                         "targets": {"attention_frac_asked": 0.60, "met": achieved / hbm_peak >= 0.60},
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH if args.variant != "simt" else None,
                         "traffic_source": "ncu capture of the attention launch at this workload's shape "
                                           "(profiles/mla_decode_tc_b32x4k_2layers.md): dram__bytes_read.sum + "
                                           "dram__bytes_write.sum per launch",
                         "algorithmic_bytes_per_launch": ATTN_BYTES_PER_LAUNCH, "us_per_launch": attn_ms * 1e3,
                         "tflops": ATTN_FLOPS_PER_LAUNCH / (attn_ms * 1e-3) * 1e-12,
                         "frac_of_measured_bf16_peak": ATTN_FLOPS_PER_LAUNCH / (attn_ms * 1e-3) * 1e-12 / tflops_peak},
            "move_kernels": move,
            "cpu_baseline": {"value": cpu_value, "unit": "tokens/s", "cores": cpu_threads, "kind": "port",
                             "sample": cpu_sample_desc},
            "e2e": {"value": None if args.skip_e2e else world * BATCH / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "copy_floor_ms": floor_ms,
                    "copies": "one H2D (q and new rows, one pinned block) and one D2H per layer, four device "
                              "buffers per direction; copy_floor_ms = the same copies with no kernels"},
            "longctx": legs.get("longctx"), "ragged": legs.get("ragged"),
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_extra_workload(args):
    """--workload ragged | longctx: one of the two multi-GPU configurations as a run of its own."""
    import torch
    import torch.distributed as dist

    import b200kv

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    if args.workload == "ragged":
        res = leg_ragged(torch, dist, b200kv, args.layers, args.steps, use_graph=not args.no_graph)
        ms = res["ms_per_run_43_layers"]
    else:
        res = leg_longctx(torch, dist, b200kv, args.layers, args.steps, args.exchange, use_graph=not args.no_graph,
                          max_ctas=args.max_ctas, tokens=args.tokens)
        ms = res["ms_per_step_43_layers"]
    if rank == 0:
        print(json.dumps({
            "metric": f"decode tokens/s ({args.workload})", "value": res["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": res["workload"]},
            "roofline": {"bound": "hbm", "achieved": res["rank0_hbm_gbs"], "peak": measured_peaks()[0], "unit": "GB/s",
                         "frac": res["rank0_frac_of_measured_hbm"], "peak_kind": res["peak_kind"],
                         "note": "rank 0's KV bytes per step over the step time, launch overhead included"},
            "detail": res,
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
    ap.add_argument("--max-ctas", type=int, default=0, help="longctx only: grid of the decode kernel (0 = one CTA per SM)")
    ap.add_argument("--tokens", type=int, default=262144, help="longctx only: length of the sequence (a multiple of 64)")
    ap.add_argument("--skip-legs", action="store_true", help="leave out the longctx and ragged legs of the default run")
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
