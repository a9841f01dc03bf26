#!/usr/bin/env python
"""Benchmark: int8 inferences/s of the lowered-graph hot path on B200, with parity, roofline and CPU baseline.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--configs all|none|a,b,..] [--impl reference]

One step = one pass of the workload's lowered graph over one batch of seeded synthetic input.
The headline workload is the single int8 Dense of the Dense sweep at its largest point
(M=131072, K=N=8192: requant shift 10, round-half-up, int8 saturation, fused bias + ReLU).

What one run prints (ONE JSON line from rank 0):

`value`        device-resident throughput of the headline (inputs already in HBM), whole job, max-over-ranks
               time.  With N > 1 GPUs every rank runs the same per-GPU batch (weak scaling, no collective).
               The K timed steps are repeated as back-to-back blocks until the region lasts about a second;
               the median block is reported, the spread beside it, and the clocks are sampled across all of it.
`parity`       a sample of the timed run's device output compared bit for bit with the CPU oracle on the same
               rows (outside the timed region).  Any mismatch makes the process exit non-zero.
`roofline`     achieved / peak for the headline kernel; also per clock (`ops_per_clk_per_sm`) so a power-capped
               run and a slow kernel can be told apart, and against a library int8 GEMM timed in this process.
`e2e`          the same metric through the model API with HOST (pinned) buffers: H2D of the inputs and D2H of
               the outputs inside the timed region, streamed in row chunks; `copy_only_ms` is the same pipeline
               with the launches left out (what the host's memory and PCIe fabric allow).
`configs`      the other benchmark configurations (small MLP, the Dense sweep, encoder block with both softmax
               modes, the three row ops, wide MLP), each with its own timing, roofline, clocks and parity.
`strong`       one batch split across the ranks by rows (`sharding.shard_rows`): Dense M=131072 and the wide MLP
               at batch 262144, per-step time max-over-ranks, with and without the final NCCL gather, and a
               parity check of the gathered result.
`cpu_baseline` the C edition of the CPU oracle on a bounded sample of the headline workload.
`--impl reference` times that CPU implementation alone (the reference's own executor is the AMD Vitis
               simulator, which cannot run here) and prints the same line shape.
"""

from __future__ import annotations

import argparse
import contextlib
import copy
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = ('dense', 'cfg1', 'cfg3_exp', 'cfg3_hccs', 'cfg4_ln', 'cfg4_sm_exp', 'cfg4_sm_hccs', 'cfg5')
SM_COUNT = 148
NOMINAL_INT8_TOPS = 4500.0

# the `configs` block: name -> (workload, overrides)
SWEEP_M = (1024, 16384, 131072)
SWEEP_KN = (1024, 4096, 8192)
CONFIG_TABLE = [('cfg1', 'cfg1', {})]
CONFIG_TABLE += [(f'cfg2_M{m}_KN{kn}', 'dense', {'m': m, 'k': kn, 'n': kn}) for m in SWEEP_M for kn in SWEEP_KN]
CONFIG_TABLE += [(n, n, {}) for n in ('cfg3_exp', 'cfg3_hccs', 'cfg4_ln', 'cfg4_sm_exp', 'cfg4_sm_hccs', 'cfg5')]
# sampled units checked against the oracle per workload kind
PARITY_UNITS = {'dense': 256, 'cfg1': 512, 'cfg3_exp': 6, 'cfg3_hccs': 6, 'cfg4_ln': 512, 'cfg4_sm_exp': 512,
                'cfg4_sm_hccs': 512, 'cfg5': 256}


# ------------------------------------------------------------------------------------------------
# workload table
# ------------------------------------------------------------------------------------------------
def build_workload(name: str, args):
    """-> dict(name, builder, inputs, units, kernel, key (for recorded DRAM traffic), desc)"""
    from aie4ml_b200 import workloads as W

    r = args.rounding
    if name == 'dense':
        M, K, N = args.m, args.k, args.n
        b, inp = W.dense_cfg2(M, K, N, rounding=r)
        return dict(name=name, builder=b, inputs=inp, units=M, kernel='dense', key=f'dense_M{M}_K{K}_N{N}',
                    desc=f'dense_cfg2 M={M} K={K} N={N} shift=10 relu bias {r}')
    if name == 'cfg1':
        batch = args.batch or 1024
        b, inp = W.mlp_cfg1(batch, rounding=r)
        return dict(name=name, builder=b, inputs=inp, units=batch, kernel='mlp', key=f'cfg1_batch{batch}',
                    desc=f'mlp_cfg1 16-64-32-32-5 batch={batch} {r}')
    if name in ('cfg3_exp', 'cfg3_hccs'):
        batch = args.batch or 4096
        b, inp = W.encoder_cfg3(batch, softmax=name.split('_')[1], rounding=r)
        return dict(name=name, builder=b, inputs=inp, units=batch, kernel='encoder', key=f'{name}_batch{batch}',
                    desc=f'encoder_cfg3 {name[5:]} batch={batch} seq=128 d=256 h=4 ffn=1024 {r}')
    if name in ('cfg4_ln', 'cfg4_sm_exp', 'cfg4_sm_hccs'):
        rows = args.batch or (1 << 20)
        op = {'cfg4_ln': 'layer_norm', 'cfg4_sm_exp': 'softmax_exp', 'cfg4_sm_hccs': 'softmax_hccs'}[name]
        b, inp = W.rowops_cfg4(rows, 1024, op, rounding=r)
        return dict(name=name, builder=b, inputs=inp, units=rows, kernel=op, key=f'{name}_rows{rows}',
                    desc=f'rowops_cfg4 {op}+add rows={rows} cols=1024 {r}')
    if name == 'cfg5':
        batch = args.batch or 262144
        b, inp = W.wide_mlp_cfg5(batch, rounding=r)
        return dict(name=name, builder=b, inputs=inp, units=batch, kernel='wide_mlp', key=f'cfg5_batch{batch}',
                    desc=f'wide_mlp_cfg5 batch={batch} {r}')
    raise SystemExit(f'unknown workload {name!r}; choose from {WORKLOADS}')


def plan_cost(plan):
    """Algorithmic bytes and integer operations of one step: per launch every operand and result once, constants
    once (an intermediate that a fused launch keeps on chip is not counted; one that passes between two launches
    is counted on both sides, since at these sizes it leaves the L2 in between)."""
    from aie4ml_b200.report import op_cost

    total_b = total_o = 0.0
    for op in plan.ops:
        c = op_cost(plan, op)
        total_b += c['bytes']
        total_o += c['ops']
    return total_b, total_o


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU every 20 ms while the timed region runs (NVML
    queries, read only; falls back to spawning nvidia-smi every 200 ms when NVML cannot be opened)."""

    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')
    REASON_BITS = {'sw_power_cap': 0x4, 'hw_slowdown': 0x8, 'sw_thermal_slowdown': 0x20, 'hw_thermal_slowdown': 0x40}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.mx, self.power, self.reasons = [], [], [], set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _nvml_handle(self):
        import pynvml
        import torch

        props = torch.cuda.get_device_properties(self.index)
        bus = f'{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0'
        pynvml.nvmlInit()
        return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())

    def _run(self):
        try:
            nv, h = self._nvml_handle()
        except Exception:
            nv = None
        while not self._stop.is_set():
            try:
                if nv is not None:
                    self.sm.append(int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                    self.mx.append(int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                    self.reasons.update(n for n, bit in self.REASON_BITS.items() if mask & bit)
                    try:
                        self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    except Exception:
                        pass
                else:
                    out = subprocess.run(['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                                          '-i', str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                    f = [x.strip() for x in out.splitlines()[0].split(',')] if out else []
                    if len(f) >= 6 and f[0].isdigit():
                        self.sm.append(int(f[0]))
                        self.mx.append(int(f[1]))
                        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
                        self.reasons.update(n for n, v in zip(names, f[2:6]) if v.lower().startswith('active'))
            except Exception:
                pass
            self._stop.wait(0.02 if nv is not None else 0.2)
        if nv is not None:
            try:
                nv.nvmlShutdown()
            except Exception:
                pass

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        return {'sm_mhz': int(np.median(self.sm)) if self.sm else None, 'sm_min_mhz': min(self.sm) if self.sm else None,
                'sm_max_mhz': max(self.mx) if self.mx else None, 'reasons': sorted(self.reasons), 'samples': len(self.sm),
                'power_w_median': round(float(np.median(self.power)), 1) if self.power else None}


# ------------------------------------------------------------------------------------------------
# peaks
# ------------------------------------------------------------------------------------------------
def measured_peaks():
    path = ROOT / 'MEASURED_PEAKS.json'
    if path.exists():
        d = json.loads(path.read_text())
        return {'hbm_gbs': float(d['hbm_gbs']), 'bf16_tflops': float(d['bf16_tflops']),
                'bf16_tflops_sustained': float(d.get('bf16_tflops_sustained', d['bf16_tflops'])), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0, 'source': 'fallback'}


def recorded_traffic():
    """DRAM bytes per launch that ncu measured (dram__bytes_read.sum + dram__bytes_write.sum), from the text summary
    `profiles/dram_traffic.txt`: lines of `key=value` fields, one capture per line.  -> {workload key: record}"""
    path = ROOT / 'profiles' / 'dram_traffic.txt'
    out = {}
    if not path.exists():
        return out
    for line in path.read_text().splitlines():
        line = line.strip()
        if not line or line.startswith('#'):
            continue
        rec = dict(f.split('=', 1) for f in line.split() if '=' in f)
        if 'workload' in rec and 'dram_bytes' in rec:
            out[rec['workload']] = rec
    return out


def int8_library_probe(seconds: float = 1.0):
    """Times the library int8 GEMM (torch._int_mm, 8192^3) back to back for about `seconds`: the int8 tensor
    throughput this GPU sustains under the same power cap, as a measured denominator.  Timing only; nothing of
    the product runs through it.  -> {'tops', 'ms', 'iters'} or None."""
    import torch

    try:
        n = 8192
        a = torch.randint(-128, 128, (n, n), dtype=torch.int8, device='cuda')
        b = torch.randint(-128, 128, (n, n), dtype=torch.int8, device='cuda')
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        iters = max(5, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
        e0.record()
        for _ in range(iters):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        del a, b
        return {'tops': 2.0 * n ** 3 / (ms * 1e-3) / 1e12, 'ms': ms, 'iters': iters, 'what': 'torch._int_mm 8192^3 back to back'}
    except Exception as exc:   # a build of torch without the int8 GEMM
        return {'tops': None, 'error': str(exc)[:120]}


# ------------------------------------------------------------------------------------------------
# timing
# ------------------------------------------------------------------------------------------------
class Dist:
    """Barrier and max-over-ranks that degrade to no-ops on one rank."""

    def __init__(self, world: int):
        self.world = world

    def barrier(self):
        import torch

        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def max(self, values):
        import torch

        if self.world == 1:
            return list(values)
        import torch.distributed as dist

        t = torch.tensor(list(values), dtype=torch.float64, device='cuda')
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]


def time_steps(run_step, steps: int, warmup: int, flush, dist: Dist, device_index: int, min_region_s: float = 1.0):
    """Warm up, then time blocks of exactly `steps` steps with CUDA events, back to back, until the region lasts
    about `min_region_s` (at least one block).  With `flush` (a buffer larger than the L2) every step gets its own
    event pair and the buffer is rewritten between steps, outside the pairs.
    -> dict(block_ms: max-over-ranks per block, local_block_ms, clocks)"""
    import torch

    for _ in range(warmup):
        run_step()
    torch.cuda.synchronize()
    # one untimed-for-the-record block to size the region
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run_step()
    e1.record()
    torch.cuda.synchronize()
    est_ms = dist.max([e0.elapsed_time(e1)])[0]
    n_blocks = int(min(max(1, math.ceil(min_region_s * 1e3 / max(est_ms, 1e-3))), 64))
    if flush is not None:
        n_blocks = max(1, min(n_blocks, 1500 // max(1, steps)))   # the flushes dominate the wall time here
    dist.barrier()
    with ClockSampler(device_index) as clocks:
        if flush is not None:
            pairs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
                     for _ in range(n_blocks)]
            for block in pairs:
                for s0, s1 in block:
                    flush.zero_()
                    s0.record()
                    run_step()
                    s1.record()
            torch.cuda.synchronize()
            local = [sum(s0.elapsed_time(s1) for s0, s1 in block) for block in pairs]
        else:
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_blocks)]
            for s0, s1 in pairs:
                s0.record()
                for _ in range(steps):
                    run_step()
                s1.record()   # one pair of events around the K steps: nothing but the steps sits between them
            torch.cuda.synchronize()
            local = [s0.elapsed_time(s1) for s0, s1 in pairs]
    dist.barrier()
    return {'block_ms': dist.max(local), 'local_block_ms': local, 'clocks': clocks.summary()}


def block_stats(block_ms, steps):
    per = sorted(b / steps for b in block_ms)
    return {'n': len(per), 'steps_per_block': steps, 'ms_per_step_median': float(np.median(per)), 'ms_per_step_min': per[0],
            'ms_per_step_max': per[-1]}


def roofline_of(plan, ms_per_step: float, clocks: dict, peaks: dict, int8_probe, single_kernel: bool):
    """Roofline record of one step: the bound is whichever of (ops / int8 tensor peak) and (bytes / HBM peak) is
    larger; `frac` = that floor / measured time."""
    bytes_step, ops_step = plan_cost(plan)
    sec = ms_per_step * 1e-3
    peak_tc = 2.0 * peaks['bf16_tflops']     # int8 dense tensor rate = 2 x the bf16 rate on this part
    t_tc, t_hbm = ops_step / (peak_tc * 1e12), bytes_step / (peaks['hbm_gbs'] * 1e9)
    mhz = clocks.get('sm_mhz') or 0
    rec = {'t_tensor_ms': t_tc * 1e3, 't_hbm_ms': t_hbm * 1e3, 'algorithmic_bytes': bytes_step, 'ops': ops_step,
           'kernel_ms': ms_per_step, 'whole_step': not single_kernel}
    if t_tc >= t_hbm:
        achieved = ops_step / sec / 1e12
        rec.update({'bound': 'tensor', 'achieved': achieved, 'peak': peak_tc, 'unit': 'TFLOP/s', 'frac': achieved / peak_tc,
                    'peak_source': f"2 x bf16_tflops (burst) of {peaks['source']} peaks: int8 rate = 2 x bf16",
                    'frac_of_2x_bf16_sustained': achieved / (2.0 * peaks['bf16_tflops_sustained']),
                    'frac_of_nominal_4500': achieved / NOMINAL_INT8_TOPS})
        if int8_probe and int8_probe.get('tops'):
            rec['peak_int8_measured'] = int8_probe['tops']
            rec['frac_of_int8_measured'] = achieved / int8_probe['tops']
        if mhz:
            rec['ops_per_clk_per_sm'] = ops_step / (sec * mhz * 1e6 * SM_COUNT)
            rec['ops_per_clk_per_sm_peak'] = 16384   # 8192 int8 MACs per clock per SM
    else:
        achieved = bytes_step / sec / 1e9
        rec.update({'bound': 'hbm', 'achieved': achieved, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                    'frac': achieved / peaks['hbm_gbs'], 'peak_source': f"hbm_gbs of {peaks['source']} peaks"})
        if ops_step:
            rec['tensor_tops'] = ops_step / sec / 1e12
        if mhz:
            rec['bytes_per_clk'] = bytes_step / (sec * mhz * 1e6)
    rec['traffic'] = None
    return rec


def parity_of(model, plan, wl, c_lib):
    """Sampled units of the plan's device outputs (left by the timed run) against the oracle.  The Dense sweep and
    the wide MLP go through the C edition (a NumPy int64 product at K = 8192 takes minutes), the rest through NumPy."""
    import torch

    from oracle import checker

    want = PARITY_UNITS.get(wl['name'], 256)
    units = checker.sample_units(wl['units'], want, tile=128, seed=wl['units'] % 9973)
    idx = torch.from_numpy(units).to(plan.device)
    got = {}
    for n in model.context.ir.logical.output_tensor_names:
        got[n] = plan.tensor_of(n).index_select(0, idx).cpu().numpy()
    use_c = wl['name'] in ('dense', 'cfg5', 'cfg3_exp', 'cfg3_hccs')
    return checker.check_sample(model.export_plan(), wl['inputs'], got, units, lib=c_lib if use_c else None)


def load_inputs(plan, graph, inputs):
    import torch

    for n in graph.input_tensor_names:
        plan.tensor_of(n).copy_(torch.from_numpy(np.ascontiguousarray(inputs[n])).to(plan.device), non_blocking=False)
    torch.cuda.synchronize()


def run_entry(name, wl_name, overrides, args, dist, local_rank, peaks, int8_probe, c_lib, traffic):
    """Build, time, check and free one configuration of the `configs` block."""
    import torch

    from aie4ml_b200 import from_graph

    sub = copy.copy(args)
    sub.batch = 0
    for k, v in overrides.items():
        setattr(sub, k, v)
    t_wall = time.perf_counter()
    wl = build_workload(wl_name, sub)
    model = from_graph(wl['builder'])
    model.build()
    plan = model.plan
    graph = model.context.ir.logical
    load_inputs(plan, graph, wl['inputs'])
    plan.capture()
    io_bytes = sum(int(np.asarray(v).nbytes) for v in wl['inputs'].values()) + \
        sum(plan.tensor_of(n).numel() * plan.tensor_of(n).element_size() for n in graph.output_tensor_names)
    fits_l2 = io_bytes <= 2 * 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if fits_l2 else None
    t = time_steps(plan.run, args.steps, args.warmup, flush, dist, local_rank, args.region_s)
    plan.check_status()
    stats = block_stats(t['block_ms'], args.steps)
    ms = stats['ms_per_step_median']
    roof = roofline_of(plan, ms, t['clocks'], peaks, int8_probe, len(plan.launches) == 1)
    rec = traffic.get(wl['key'])
    if rec is not None and len(plan.launches) == 1:
        roof['traffic'] = float(rec['dram_bytes'])
    parity = parity_of(model, plan, wl, c_lib)
    entry = {'name': name, 'workload': wl['desc'], 'units_per_step': wl['units'], 'value': dist.world * wl['units'] / (ms * 1e-3),
             'unit': 'inferences/s', 'ms_per_step': ms, 'blocks': stats, 'launches_per_step': len(plan.launches),
             'roofline': roof, 'clocks': t['clocks'], 'parity': parity, 'fused': plan.fused,
             'l2': 'flushed between steps' if fits_l2 else 'working set exceeds the L2',
             'wall_s': round(time.perf_counter() - t_wall, 1)}
    del plan, model, wl, flush
    torch.cuda.empty_cache()
    return entry


# ------------------------------------------------------------------------------------------------
# strong scaling: one batch split across the ranks by rows
# ------------------------------------------------------------------------------------------------
def strong_entry(label, wl_name, overrides, full_inputs, args, dist, rank, local_rank, c_lib):
    """Rank r builds the plan for ITS rows [r*M/G, (r+1)*M/G) of one batch and loads them; per-step time is the
    max over ranks, once with the forward pass alone and once followed by the NCCL gather of the outputs on the
    same stream.  Rank 0 checks sampled rows of the gathered result against the oracle."""
    import torch

    from aie4ml_b200 import from_graph
    from aie4ml_b200.sharding import gather_outputs, shard_rows
    from oracle import checker

    world = dist.world
    sub = copy.copy(args)
    sub.batch = 0
    for k, v in overrides.items():
        setattr(sub, k, v)
    total = sub.m if wl_name == 'dense' else overrides['batch']
    lo, hi = shard_rows(total, rank, world)
    if wl_name == 'dense':
        sub.m = hi - lo
    else:
        sub.batch = hi - lo
    wl = build_workload(wl_name, sub)     # constants are drawn before the inputs: identical on every rank
    model = from_graph(wl['builder'])
    model.build()
    plan = model.plan
    graph = model.context.ir.logical
    load_inputs(plan, graph, {n: full_inputs[n][lo:hi] for n in graph.input_tensor_names})
    plan.capture()
    out_name = list(graph.output_tensor_names)[0]

    def step_plain():
        plan.run()

    gathered = {}

    def step_gather():
        plan.run()
        gathered['y'] = gather_outputs(plan.tensor_of(out_name), total) if world > 1 else plan.tensor_of(out_name)

    res = {}
    for key, fn in (('forward', step_plain), ('forward_gather', step_gather)):
        t = time_steps(fn, args.steps, args.warmup, None, dist, local_rank, min(args.region_s, 0.5))
        stats = block_stats(t['block_ms'], args.steps)
        res[key] = {'ms_per_step': stats['ms_per_step_median'], 'value': total / (stats['ms_per_step_median'] * 1e-3),
                    'blocks': stats, 'clocks': t['clocks']}
    plan.check_status()
    parity = None
    if rank == 0:
        units = checker.sample_units(total, 256, tile=128, seed=world)
        # the shard boundaries themselves: last row of one rank, first of the next
        edges = sorted({r for g in range(world) for r in shard_rows(total, g, world) if 0 < r < total} |
                       {r - 1 for g in range(world) for r in shard_rows(total, g, world) if 0 < r <= total})
        units = np.unique(np.concatenate([units, np.array(edges, dtype=np.int64)]))
        idx = torch.from_numpy(units).to(plan.device)
        got = {out_name: gathered['y'].index_select(0, idx).cpu().numpy()}
        # the exported plan does not depend on the number of rows: the shard's plan evaluates rows of the full batch
        parity = checker.check_sample(model.export_plan(), {n: full_inputs[n] for n in graph.input_tensor_names}, got,
                                      units, lib=c_lib)
    entry = {'name': label, 'workload': wl['desc'], 'total_units': total, 'units_per_rank': hi - lo, 'scaling': 'strong',
             'launches_per_step': len(plan.launches), **res, 'gather_bytes_per_step': int(total) * int(plan.tensor_of(out_name)[0].numel()),
             'parity': parity}
    del plan, model, wl, gathered
    torch.cuda.empty_cache()
    return entry


# ------------------------------------------------------------------------------------------------
# CPU baseline and the reference arm (the C edition of the oracle; the only legs that TIME oracle/)
# ------------------------------------------------------------------------------------------------
def cpu_baseline(wl, plan_export, c_lib, c_desc, target_seconds: float = 12.0):
    from oracle import checker

    cores = int(c_lib.orc_num_threads())
    units = wl['units']
    probe = max(1, min(units, 48))
    take = lambda rows: {k: v[:rows] for k, v in wl['inputs'].items()}
    _, t = checker.run_plan_c(c_lib, plan_export, take(probe))
    _, t = checker.run_plan_c(c_lib, plan_export, take(probe))      # second call: pages and threads are warm
    rows = probe
    # grow the sample until it costs about `target_seconds` (fixed costs such as packing the weights make the first
    # estimates pessimistic), or covers the whole workload
    for _ in range(4):
        rows = int(max(probe, min(units, rows * target_seconds / max(t, 1e-6))))
        _, t = checker.run_plan_c(c_lib, plan_export, take(rows))
        if rows >= units or t >= target_seconds / 3:
            break
    return {'value': rows / t, 'unit': 'inferences/s', 'cores': cores, 'kind': 'port',
            'sample': f'first {rows} of {units} units of the workload, C/OpenMP oracle ({c_desc}), {t:.2f} s'}


def headline_config(wl, world: int):
    """The `config` object of the JSON line: what is run, independent of how (both arms print the same one)."""
    io = sum(int(np.asarray(v).nbytes) for v in wl['inputs'].values())
    return {'workload': wl['desc'], 'per_gpu_units': wl['units'], 'sharding': f'batch rows x{world}, no collective',
            'l2': 'inputs exceed the 126 MB L2' if io > 126e6 else 'flushed between steps (256 MB write), one event pair per step'}


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    from aie4ml_b200 import from_graph
    from oracle import checker

    wl = build_workload(args.workload, args)
    plan = from_graph(wl['builder']).export_plan()
    lib, desc = checker.load_c(native=True)
    cores = int(lib.orc_num_threads())
    take = lambda rows: {k: v[:rows] for k, v in wl['inputs'].items()}
    probe = max(1, min(wl['units'], 48))
    checker.run_plan_c(lib, plan, take(probe))
    _, t = checker.run_plan_c(lib, plan, take(probe))
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows = int(max(probe, min(wl['units'], probe * min(budget, 20.0) / max(t, 1e-6))))
    for _ in range(args.warmup):
        checker.run_plan_c(lib, plan, take(rows))
    t0 = time.perf_counter()
    spent = 0.0
    for _ in range(args.steps):
        spent += checker.run_plan_c(lib, plan, take(rows))[1]
    wall = time.perf_counter() - t0
    value = rows * args.steps / spent
    sample = f'each step = first {rows} of {wl["units"]} units, C/OpenMP oracle ({desc}), {cores} threads'
    print(json.dumps({
        'impl': 'reference', 'metric': 'int8 inferences/s', 'value': value, 'unit': 'inferences/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * wall / args.steps, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'int8', 'data': 'synthetic',
        'config': headline_config(wl, world),
        'cpu_baseline': {'value': value, 'unit': 'inferences/s', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': 'inferences/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'note': "the reference's own executor is the AMD Vitis x86 simulator, unavailable on this box; this arm is "
                'the CPU restatement of its kernels',
    }))


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='dense', choices=WORKLOADS)
    ap.add_argument('--m', type=int, default=131072)
    ap.add_argument('--k', type=int, default=8192)
    ap.add_argument('--n', type=int, default=8192)
    ap.add_argument('--batch', type=int, default=0)
    ap.add_argument('--rounding', default='half_up', choices=['half_up', 'conv_even', 'floor', 'sym_inf'])
    ap.add_argument('--configs', default=None,
                    help="'all', 'none' or a comma list of names from the configs table (default: all on one GPU, none on several)")
    ap.add_argument('--no-strong', action='store_true', help='skip the strong-scaling block')
    ap.add_argument('--no-cpu', action='store_true', help='skip the CPU baseline leg')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-probe', action='store_true', help='skip the library int8 GEMM probe')
    ap.add_argument('--e2e-chunks', type=int, default=0, help='row chunks of the end-to-end pipeline (0 = automatic)')
    ap.add_argument('--region-s', type=float, default=1.0, help='length of each timed region in seconds (blocks of --steps steps)')
    ap.add_argument('--no-graph', action='store_true')
    ap.add_argument('--no-numa', action='store_true', help='do not place the pinned host buffers next to the GPU')
    ap.add_argument('--algo', type=int, default=0, help='dense kernel: 0 auto, 1 simt, 2 tcgen05')
    ap.add_argument('--dense-panel-mib', type=int, default=None,
                    help='tcgen05 Dense: MiB of weights per column panel of the tile order (library default 32; 0 = one panel)')
    ap.add_argument('--no-dense-ln', action='store_true',
                    help='keep Dense and Add + LayerNorm as two launches (the single kernel for 256-wide layers is the default)')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup

    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))

    if args.impl == 'reference':
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as tdist

    from aie4ml_b200 import from_graph
    from oracle import checker

    if not torch.cuda.is_available():
        raise SystemExit('bench.py: no CUDA device visible; the product path has no CPU fallback '
                         '(use --impl reference for the CPU arm).')
    torch.cuda.set_device(local_rank)
    if world > 1:
        tdist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
    dist = Dist(world)
    peaks = measured_peaks()
    traffic = recorded_traffic()
    c_lib, c_desc = checker.load_c(native=True)
    if args.dense_panel_mib is not None:
        from aie4ml_b200 import lib as a4c

        a4c.check(a4c.load().a4c_set_option(a4c.OPT_DENSE_PANEL_MIB, args.dense_panel_mib), 'a4c_set_option')
    if args.no_dense_ln:
        from aie4ml_b200 import lib as a4c

        a4c.check(a4c.load().a4c_set_option(a4c.OPT_DENSE_LN_PATH, 1), 'a4c_set_option')

    wl = build_workload(args.workload, args)
    model = from_graph(wl['builder'])
    model.context.aie_config['DenseAlgo'] = args.algo
    model.build()
    plan = model.plan
    graph = model.context.ir.logical
    in_names, out_names = list(graph.input_tensor_names), list(graph.output_tensor_names)

    # pinned host buffers (the e2e leg copies from / to these every step), placed on the NUMA node nearest to this
    # rank's GPU unless --no-numa
    from aie4ml_b200.streaming import near_gpu

    with (contextlib.nullcontext() if args.no_numa else near_gpu(local_rank)) as numa:
        host_in = {n: torch.empty(wl['inputs'][n].shape, dtype=torch.from_numpy(wl['inputs'][n][:0]).dtype).pin_memory()
                   for n in in_names}
        host_out = {n: torch.empty(plan.tensor_of(n).shape, dtype=plan.tensor_of(n).dtype).pin_memory() for n in out_names}
        for n in in_names:
            host_in[n].copy_(torch.from_numpy(np.ascontiguousarray(wl['inputs'][n])))
        for n in out_names:
            host_out[n].zero_()
    placement = numa.describe() if numa is not None else {'requested': False}
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())
    for n in in_names:
        plan.tensor_of(n).copy_(host_in[n], non_blocking=True)
    torch.cuda.synchronize()

    launches_per_step = len(plan.launches)
    if not args.no_graph:
        plan.capture()   # one replay per step: the host's per-launch cost stays out of the device timing

    # ---- library int8 GEMM probe (a measured denominator; before the headline so both see a warm GPU) ----------
    int8_probe = None if args.no_probe else int8_library_probe(args.region_s)

    # ---- device-resident timing --------------------------------------------------------------
    # L2 rule: a working set above the 126 MB L2 evicts itself between steps; a smaller one is flushed by writing a
    # 256 MB buffer between steps, and then every step gets its own event pair so the flush stays outside the timing.
    fits_l2 = h2d <= 126e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if fits_l2 else None
    timed = time_steps(plan.run, args.steps, args.warmup, flush, dist, local_rank, args.region_s)
    plan.check_status()
    stats = block_stats(timed['block_ms'], args.steps)
    ms_per_step = stats['ms_per_step_median']
    value = world * wl['units'] / (ms_per_step * 1e-3)
    local_ms_per_step = float(np.median(timed['local_block_ms'])) / args.steps

    # ---- parity of what the timed run left in the output buffers -------------------------------
    parity = parity_of(model, plan, wl, c_lib)

    # ---- end-to-end timing: host pinned buffers -> H2D -> launches -> D2H ----------------------
    e2e = None
    if not args.no_e2e:
        # The host batch is cut into chunks of rows; copy-in, launches and copy-out of different chunks
        # overlap on three streams (aie4ml_b200.streaming.HostPipeline).  All of it is inside the timed region.
        # Many ranks share one host's memory and PCIe fabric: fewer, larger copies then queue better.
        want_chunks = args.e2e_chunks or (16 if world <= 2 else 8)
        chunks = want_chunks if (wl['units'] % want_chunks == 0 and wl['units'] // want_chunks >= 256) else 1
        if chunks > 1:
            sub = copy.copy(args)
            sub.m = args.m // chunks
            sub.batch = wl['units'] // chunks
            wl_c = build_workload(args.workload, sub)
            model_c = from_graph(wl_c['builder'])
            model_c.context.aie_config['DenseAlgo'] = args.algo
            model_c.build()
            pipe = model_c.pipeline(3)
            del wl_c
        else:
            pipe = model.pipeline(1)

        def e2e_time(fn, k):
            for _ in range(2):
                fn()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(k):
                fn()
            e1.record()
            torch.cuda.synchronize()
            dist.barrier()
            return dist.max([e0.elapsed_time(e1)])[0] / k

        k2 = max(3, min(args.steps, 10))
        e2e_ms = e2e_time(lambda: pipe.run(host_in, host_out), k2)
        pipe.plans[0].check_status()
        same = all(bool(torch.equal(host_out[n], plan.tensor_of(n).cpu())) for n in out_names)
        copy_ms = e2e_time(lambda: pipe.run(host_in, host_out, launches=False), k2)
        e2e = {'value': world * wl['units'] / (e2e_ms * 1e-3), 'unit': 'inferences/s', 'h2d_bytes_per_step': h2d,
               'd2h_bytes_per_step': d2h, 'ms_per_step': e2e_ms, 'chunks': chunks,
               'gpu_launches_per_step': pipe.launches_per_chunk * chunks, 'equals_device_resident_run': same,
               'copy_only_ms': copy_ms, 'fraction_of_copy_only': copy_ms / e2e_ms if e2e_ms > 0 else None,
               'host_gb_per_s_all_ranks': world * (h2d + d2h) / (e2e_ms * 1e-3) / 1e9, 'host_buffers': placement}
        del pipe

    # ---- roofline of the headline kernel ----------------------------------------------------------
    roof = roofline_of(plan, local_ms_per_step, timed['clocks'], peaks, int8_probe, launches_per_step == 1)
    rec = traffic.get(wl['key'])
    if rec is not None and launches_per_step == 1:
        roof['traffic'] = float(rec['dram_bytes'])
        roof['traffic_source'] = 'ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload'

    # ---- strong scaling block (every N, so that the N = 1 time is on record beside the others) ----------------
    strong = []
    if not args.no_strong and args.workload == 'dense':
        strong.append(strong_entry('cfg2_M131072_KN8192_rows_split', 'dense', {'m': args.m, 'k': args.k, 'n': args.n},
                                   wl['inputs'], args, dist, rank, local_rank, c_lib))
        from aie4ml_b200 import workloads as W

        _, cfg5_inputs = W.wide_mlp_cfg5(262144, rounding=args.rounding)
        strong.append(strong_entry('cfg5_batch262144_rows_split', 'cfg5', {'batch': 262144}, cfg5_inputs, args, dist,
                                   rank, local_rank, c_lib))
        del cfg5_inputs

    # ---- the other configurations -----------------------------------------------------------------
    which = args.configs if args.configs is not None else ('all' if world == 1 else 'none')
    configs = []
    if which != 'none':
        names = None if which == 'all' else set(which.split(','))
        for name, wl_name, overrides in CONFIG_TABLE:
            if names is not None and name not in names:
                continue
            if wl_name == args.workload == 'dense' and (overrides['m'], overrides['k'], overrides['n']) == (args.m, args.k, args.n):
                configs.append({'name': name, 'workload': wl['desc'], 'see': 'headline', 'value': value, 'ms_per_step': ms_per_step,
                                'roofline': {k: roof[k] for k in ('bound', 'achieved', 'peak', 'frac')}, 'parity': parity,
                                'clocks': timed['clocks']})
                continue
            configs.append(run_entry(name, wl_name, overrides, args, dist, local_rank, peaks, int8_probe, c_lib, traffic))

    bad = parity['mismatches'] + sum(c['parity']['mismatches'] for c in configs) + \
        sum(s['parity']['mismatches'] for s in strong if s.get('parity'))
    if rank == 0:
        line = {
            'metric': 'int8 inferences/s', 'value': value, 'unit': 'inferences/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'int8', 'data': 'synthetic',
            'config': headline_config(wl, world),
            'execution': {'cuda_graph': plan.graph_exec is not None, 'fused': plan.fused,
                          'timing': f"median of {stats['n']} back-to-back blocks of {args.steps} steps, CUDA events"},
            'blocks': stats, 'parity': parity, 'roofline': roof, 'clocks': timed['clocks'],
            'gpu_launches': launches_per_step * args.steps * stats['n'], 'gpu_launches_per_step': launches_per_step,
            'int8_library_probe': int8_probe,
        }
        if e2e is not None:
            line['e2e'] = e2e
        if strong:
            line['strong'] = strong
        if configs:
            line['configs'] = configs
        if not args.no_cpu:
            line['cpu_baseline'] = cpu_baseline(wl, model.export_plan(), c_lib, c_desc)
        print(json.dumps(line))
    if world > 1:
        tdist.barrier()
        tdist.destroy_process_group()
    if bad:
        raise SystemExit(f'bench.py: {bad} output values differ from the CPU oracle')


if __name__ == '__main__':
    main()
