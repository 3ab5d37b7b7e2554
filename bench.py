#!/usr/bin/env python
"""Benchmark of the depthwise 3x3x3 channels-last fp16 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--channels 8,16,...]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A STEP is one pass over the headline sweep: for every C in {8, 16, 32, 64, 128}, DWConv of a
(1, C, 350, 350, 128) fp16 channels_last_3d volume followed by DWConvWGRAD of the same volume against
an independent gradient (seeded synthetic N(0,1) data, weights U(+-1/sqrt(27))).  With N GPUs every rank
runs the sweep on its own sample (weak scaling) and the fp32 [27][C] weight gradients of a step are summed
once per step - by the library's own push/flag/sum kernel over peer memory (--allreduce push, the default) or by
NCCL - the only exchange the sample-sharded path has.

`value` = algorithmic bytes of all ranks / max-over-ranks device time; algorithmic bytes are 4*V*C per
operator call (read x + write y, or read x + read grad; V = 350*350*128 voxels).
The JSON line also carries: `roofline` (the kernel with the largest share of the timed region, bytes /
CUDA-event time against the measured HBM peak), `detail` (per operator and C: ms mean / median / min, GB/s,
fraction, ratio to torch.clone, the packed-half accumulate mode, two small-shape latencies), `e2e` (the same sweep
through the host-buffer operator DWConvStepHost, host<->device copies inside the timed region), `cpu_baseline`
(torch CPU depthwise conv3d, the check the reference's tests use, on a bounded sample), `clocks` (SM clock and
throttle reasons sampled through NVML during the timed region), at one GPU `reference_triton_on_this_gpu` (the
reference's own Triton kernels from baseline/_ref timed on the same tensors) with `vs_reference_triton` (the
speed-ups), and - at every N - the two strong-scaling workloads as sub-records:
`dshard` = one (1,128,1400,350,128) volume sharded along H over the ranks with halo exchange (BASELINE configs[3]) and
`dpstep` = a batch of 8 x (32,350,350,128) samples split by sample (configs[4]), each with its per-rank breakdown,
so that strong-scaling efficiency can be computed from the lines of a 1/2/4/8-GPU series alone; at one GPU also
`fused` = the record of --workload fused (below).

--workload dshard | dpstep | fused run one of the other workloads alone (`fused` = DWConvAddStats and DWConvBNReLU
against the unfused and the reference two-operator chains, one GPU).

`--impl reference` times the CPU arm alone (rank 0 only, all host cores): torch conv3d(groups=C) forward + weight
gradient over the same five-C sweep, every volume cut to a slab of h-planes so that a step stays near a second; the
slab times are scaled to the full volumes by plane count (conv3d's cost is proportional to it).
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPE = (350, 350, 128)  # kerops H, W, D = torch dims 2, 3, 4
VOX = SHAPE[0] * SHAPE[1] * SHAPE[2]
ALL_CHANNELS = [8, 16, 32, 64, 128]
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the kernels the library chooses by itself, from one
# `ncu --set full` capture on (1, C, 100, 350, 128) volumes, scaled by 350/100 planes (traffic grows in proportion to
# the planes a launch processes).  Bytes per (1,C,350,350,128) launch; None where no capture has been taken.
NCU_TRAFFIC = {
    ('fprop', 8): int((0.079657 + 0.026334) * 3.5e9),
    ('wgrad', 8): int((0.151532 + 0.004746) * 3.5e9),
    ('fprop', 32): int((0.290739 + 0.246126) * 3.5e9),
    ('wgrad', 32): int((0.577468 + 0.004517) * 3.5e9),
    ('fprop', 128): int((1.314928 + 1.107812) * 3.5e9),
    ('wgrad', 128): int((2.545495 + 0.007897) * 3.5e9),
}


def set_planes(h):
    global SHAPE, VOX
    SHAPE = (h, SHAPE[1], SHAPE[2])
    VOX = SHAPE[0] * SHAPE[1] * SHAPE[2]


def algorithmic_bytes(C, n_samples=1):
    return 4 * VOX * C * n_samples


def measured_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return FALLBACK_HBM_GBS, 'fallback'


# ----------------------------------------------------------------------------------------------------
# clocks through NVML (read-only)
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x4: 'sw_power_cap', 0x8: 'hw_slowdown', 0x20: 'sw_thermal_slowdown', 0x40: 'hw_thermal_slowdown',
               0x80: 'hw_power_brake_slowdown', 0x2: 'applications_clocks_setting', 0x10: 'sync_boost'}

    def __init__(self, torch_device):
        self.samples, self.reasons, self.err = [], set(), None
        self.max_mhz = None
        self._stop = threading.Event()
        self._recording = threading.Event()
        self._thread = None
        self.period_s = 0.01
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self.nv = pynvml
            props = torch.cuda.get_device_properties(torch_device)
            handle = None
            uuid = getattr(props, 'uuid', None)
            if uuid is not None:
                try:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(('GPU-' + str(uuid)).encode())
                except Exception:
                    handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(torch_device.index or 0)
            self.h = handle
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # no NVML: report it instead of failing the benchmark
            self.err = f'{type(e).__name__}: {e}'

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                if self._recording.is_set():
                    self.samples.append(mhz)
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception as e:
                self.err = f'{type(e).__name__}: {e}'
                return
            time.sleep(self.period_s)

    def start(self):
        """Starts polling.  Call it BEFORE the warm-up: the first NVML queries of a process stall its CUDA
        launches for milliseconds (more with several ranks on one node); samples are kept only after begin()."""
        if self.err is None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def begin(self):
        """Marks the start of the timed region."""
        self.samples, self.reasons = [], set()
        self._recording.set()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        if not self.samples and self.err is None:  # timed region shorter than one polling period
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            except Exception as e:
                self.err = f'{type(e).__name__}: {e}'
        out = {'sm_mhz': statistics.median(self.samples) if self.samples else None, 'sm_max_mhz': self.max_mhz,
               'reasons': sorted(self.reasons), 'samples': len(self.samples)}
        if self.err:
            out['error'] = self.err
        return out


# ----------------------------------------------------------------------------------------------------
# CPU arm: torch depthwise conv3d on the host cores (the reference tests' own check, test_conv.py:25,60-72)
# ----------------------------------------------------------------------------------------------------
def cpu_threads():
    """Host cores this process may use (torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm undoes that)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_slab_planes(C):
    """h-planes of the CPU arm's slab for channel count C: the full 350 at C = 8, halved for every doubling of C, so
    that every C costs about the same CPU time."""
    return max(8, min(SHAPE[0], (SHAPE[0] * 8) // C))


def make_cpu_inputs(C, planes, seed=0):
    import torch

    g = torch.Generator().manual_seed(seed)
    _, W, D = SHAPE
    x = torch.randn(1, planes, W, D, C, generator=g, dtype=torch.float32).to(torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(1, planes, W, D, C, generator=g, dtype=torch.float32).to(torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g) * 2 - 1) / math.sqrt(27)).to(torch.float16)
    return x, grad, w


def cpu_step(x, grad, w, dtype):
    """fprop + weight gradient of one volume with torch on the CPU; returns (y, dw)."""
    import torch
    import torch.nn.functional as F
    from oracle import torch_oracle

    C = x.shape[1]
    wt = torch_oracle.to_torch_weight(w).to(dtype).requires_grad_(True)
    y = F.conv3d(x.to(dtype), wt, None, stride=1, padding=1, groups=C)
    y.backward(grad.to(dtype))
    return y.detach().to(torch.float16), wt.grad


def time_cpu_arm(channels, steps, warmup, min_seconds=0.0):
    """The five-C sweep on the host cores, on slabs.  Returns a dict: seconds per FULL sweep step (median over the
    steps of the sum over C of slab time x 350 / slab planes), the dtype used (the faster of fp32 / fp16 at the first
    C), per-C slab planes and seconds, CPU seconds spent in timed steps and their number."""
    import torch

    torch.set_num_threads(cpu_threads())
    data = {C: make_cpu_inputs(C, cpu_slab_planes(C)) for C in channels}
    C0 = channels[0]
    best = None
    for dtype in (torch.float32, torch.float16):
        try:
            cpu_step(*data[C0], dtype)
            t0 = time.perf_counter()
            cpu_step(*data[C0], dtype)
            dt = time.perf_counter() - t0
            if best is None or dt < best[0]:
                best = (dt, dtype)
        except Exception:
            continue
    if best is None:
        raise RuntimeError('torch CPU conv3d failed in both fp32 and fp16')
    dtype = best[1]
    for _ in range(warmup):
        for C in channels:
            cpu_step(*data[C], dtype)
    totals, per_c, spent = [], {C: [] for C in channels}, 0.0
    while len(totals) < steps or (spent < min_seconds and len(totals) < 200):
        tot = 0.0
        for C in channels:
            t0 = time.perf_counter()
            cpu_step(*data[C], dtype)
            dt = time.perf_counter() - t0
            spent += dt
            per_c[C].append(dt)
            tot += dt * SHAPE[0] / cpu_slab_planes(C)
        totals.append(tot)
    return {'sec_per_step': statistics.median(totals), 'dtype': str(dtype).replace('torch.', ''), 'spent': spent,
            'n': len(totals), 'cores': torch.get_num_threads(),
            'per_c': {str(C): {'planes': cpu_slab_planes(C), 'slab_s': round(statistics.median(per_c[C]), 4)}
                      for C in channels}}


def sweep_workload(channels, world):
    return (f'configs[1]+[2]: DWConv then DWConvWGRAD on (1,C,{SHAPE[0]},350,128) fp16 channels_last_3d for C in '
            + ','.join(map(str, channels)) + '; one sample per GPU')


def sweep_config(channels, world):
    """The `config` object both arms print (identical for the same flags)."""
    return {'workload': sweep_workload(channels, world),
            'l2': 'inputs larger than L2 (smallest tensor 251 MB; 31 GB touched per step)',
            'parallelism': f'dp{world}' if world > 1 else 'single'}


def cpu_sample_text(r, channels):
    return ('the same five-C sweep on slabs of the volumes (h-planes per C: '
            + ', '.join(f"{C}: {r['per_c'][str(C)]['planes']}" for C in channels)
            + f"), torch CPU conv3d(groups=C) forward + weight gradient in {r['dtype']}; slab times scaled to 350 planes; "
              f"median of {r['n']} steps ({r['spent']:.1f} s of CPU work)")


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    world = int(os.environ.get('WORLD_SIZE', '1'))
    r = time_cpu_arm(args.channels, args.steps, max(1, args.warmup))
    nbytes = sum(2 * algorithmic_bytes(C) for C in args.channels)
    value = nbytes / r['sec_per_step'] / 1e9
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': round(value, 3), 'unit': 'GB/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(r['sec_per_step'] * 1e3, 2),
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': r['dtype'], 'data': 'synthetic',
        'config': sweep_config(args.channels, world),
        'cpu_baseline': {'value': round(value, 3), 'unit': 'GB/s', 'cores': r['cores'], 'kind': 'port',
                         'sample': cpu_sample_text(r, args.channels)},
        'e2e': {'value': round(value, 3), 'unit': 'GB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0, 'detail': r['per_c'],
    }
    print(json.dumps(line), flush=True)


METRIC = 'DWConv + DWConvWGRAD algorithmic HBM GB/s at (1,C,350,350,128) fp16 channels_last_3d'


# ----------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------
def make_reducer(args, numel, world):
    """The library's one-kernel all-reduce over peer memory, or None for NCCL's (also when the peer mappings
    cannot be set up on this machine)."""
    if world == 1 or args.allreduce != 'push':
        return None
    import torch.distributed as dist

    from kerops_b200 import dist as kd

    red, ok = None, 1
    try:
        red = kd.GradPushAllReduce(numel)
    except Exception as e:  # e.g. no CUDA IPC between the ranks
        print(f'bench: peer-memory all-reduce unavailable ({type(e).__name__}: {e}); using NCCL', file=sys.stderr)
        ok = 0
    import torch

    flag = torch.tensor([ok], device='cuda')
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return red if int(flag.item()) == 1 else None


def make_gpu_inputs(C, device, seed):
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    H, W, D = SHAPE
    x = torch.randn(1, H, W, D, C, generator=g, device=device, dtype=torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(1, H, W, D, C, generator=g, device=device, dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device=device) * 2 - 1) / math.sqrt(27)).to(torch.float16)
    return x, grad, w


class Ctx:
    """One rank of the benchmark: device, process group."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        from kerops_b200 import _lib

        self.world = int(os.environ.get('WORLD_SIZE', '1'))
        self.rank = int(os.environ.get('RANK', '0'))
        self.local = int(os.environ.get('LOCAL_RANK', '0'))
        if self.world != args.gpus and self.world > 1:
            raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={self.world}')
        if not torch.cuda.is_available():
            raise SystemExit('bench.py needs a CUDA device: kerops_b200 has no CPU path')
        self.dev = torch.device('cuda', self.local)
        torch.cuda.set_device(self.dev)
        _lib.load()
        if self.world > 1:
            # NCCL may print a version banner on stdout when it creates its communicator; stdout carries the one
            # JSON line only, so file descriptor 1 points at stderr until the first collective has run
            sys.stdout.flush()
            saved = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group('nccl', device_id=self.dev)
                t = torch.zeros(1, device=self.dev)
                dist.all_reduce(t)
                torch.cuda.synchronize()
            finally:
                sys.stdout.flush()
                os.dup2(saved, 1)
                os.close(saved)

    def barrier(self):
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return ms
        t = torch.tensor([ms], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather_rows(self, row):
        """One list of floats per rank -> list of rows (rank order) on every rank."""
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return [list(row)]
        t = torch.tensor(row, device=self.dev, dtype=torch.float64)
        out = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(out, t)
        return [[float(v) for v in o.tolist()] for o in out]

    def close(self):
        import torch.distributed as dist

        if self.world > 1:
            dist.destroy_process_group()


def reducer_name(reducer, world):
    return ('push kernel over peer memory' if reducer is not None else 'nccl') if world > 1 else None


def breakdown(ctx, names, events):
    """events: one tuple of len(names)+1 CUDA events per timed step.  Per phase: the mean over the steps of every
    rank, ms, in rank order."""
    n = len(names)
    means = [statistics.mean(ev[i].elapsed_time(ev[i + 1]) for ev in events) for i in range(n)]
    rows = ctx.gather_rows(means)
    return {name: [round(r[i], 4) for r in rows] for i, name in enumerate(names)}


def small_shape_latency(dev, triton_ops):
    """Microseconds per call on two small shapes of the reference's test lattice, where a call is launch-bound:
    200 back-to-back calls between two events."""
    import torch

    from kerops_b200.ops.conv import DWConv, DWConvWGRAD

    out = {}
    for (N, C, H, W, D) in [(1, 8, 16, 16, 8), (2, 32, 13, 32, 7)]:
        g = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(N, H, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3)
        gr = torch.randn(N, H, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3)
        w = ((torch.rand(3, 3, 3, C, generator=g, device=dev) * 2 - 1) / math.sqrt(27)).to(torch.float16)
        row = {}
        fns = [('fprop_us', lambda: DWConv(x, w)), ('wgrad_us', lambda: DWConvWGRAD(x, gr))]
        if triton_ops is not None:
            fns += [('reference_fprop_us', lambda: triton_ops[0](x, w)), ('reference_wgrad_us', lambda: triton_ops[1](x, gr))]
        for name, fn in fns:
            try:
                for _ in range(10):
                    fn()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(200):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                row[name] = round(e0.elapsed_time(e1) / 200 * 1e3, 2)
            except Exception as e:
                row[name] = f'{type(e).__name__}'
        out[f'({N},{C},{H},{W},{D})'] = row
    return out


def sweep_record(args, ctx):
    """The headline sweep; returns the JSON line as a dict (rank 0) or None."""
    import torch
    import torch.distributed as dist

    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConv, _launch

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    channels = args.channels
    data = {C: make_gpu_inputs(C, dev, seed=1000 * rank + C) for C in channels}
    ws = {C: _launch.wgrad_workspace(data[C][0]) for C in channels}
    # one bucket for the fp32 weight gradients of a step: a single all-reduce per step when sharded by sample
    bucket = torch.empty(27 * sum(channels), dtype=torch.float32, device=dev)
    slot, off = {}, 0
    for C in channels:
        slot[C] = bucket[off:off + 27 * C]
        off += 27 * C

    reducer, bucket_out = make_reducer(args, bucket.numel(), world), torch.empty_like(bucket)

    def step(events=None):
        for C in channels:
            x, grad, w = data[C]
            if events is not None:
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record()
            y = DWConv(x, w)
            if events is not None:
                e1.record()
            dw32, dw16 = _launch.wgrad(x, grad, want_f16=(world == 1), workspace=ws[C], out_f32=slot[C])
            if events is not None:
                e2.record()
                events.append((C, e0, e1, e2))
            del y
        if world > 1:
            if reducer is not None:
                reducer(bucket, out=bucket_out)
            else:
                dist.all_reduce(bucket)

    sampler = ClockSampler(dev)
    sampler.start()
    for _ in range(args.warmup):
        step()
    ctx.barrier()
    sampler.begin()
    events = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        step(events)
    t_end.record()
    ctx.barrier()
    clocks = sampler.stop()
    total_ms = ctx.max_over_ranks(t_start.elapsed_time(t_end))
    status = _lib.device_status()

    peak, peak_kind = measured_peak()
    detail = {'fprop': {}, 'wgrad': {}}
    tot = {'fprop': [0.0, 0.0], 'wgrad': [0.0, 0.0]}  # ms, bytes
    for C in channels:
        f_all = [e0.elapsed_time(e1) for (c, e0, e1, e2) in events if c == C]
        w_all = [e1.elapsed_time(e2) for (c, e0, e1, e2) in events if c == C]
        for kind, all_ms in (('fprop', f_all), ('wgrad', w_all)):
            ms = statistics.mean(all_ms)
            gbs = algorithmic_bytes(C) / (ms * 1e-3) / 1e9
            detail[kind][str(C)] = {'ms': round(ms, 4), 'ms_median': round(statistics.median(all_ms), 4),
                                    'ms_min': round(min(all_ms), 4), 'gbs': round(gbs, 1),
                                    'frac': round(gbs / peak, 4), 'frac_of_nominal_8000': round(gbs / 8000.0, 4)}
            tot[kind][0] += ms
            tot[kind][1] += algorithmic_bytes(C)

    def timeit(fn, reps=5):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    # torch.clone of the same tensors, the comparator the reference's README uses; and the forward pass in the
    # packed-half accumulate mode (ACCTYPE='float16')
    clone = {}
    for C in channels:
        x, _, w = data[C]
        ms = timeit(lambda: x.clone())
        clone[str(C)] = {'ms': round(ms, 4), 'gbs': round(algorithmic_bytes(C) / (ms * 1e-3) / 1e9, 1)}
        for kind in ('fprop', 'wgrad'):
            detail[kind][str(C)]['x_clone'] = round(detail[kind][str(C)]['ms'] / ms, 3)
        try:
            ms16 = timeit(lambda: DWConv(x, w, ACCTYPE='float16'))
            detail['fprop'][str(C)]['acc_float16_ms'] = round(ms16, 4)
            detail['fprop'][str(C)]['acc_float16_frac'] = round(algorithmic_bytes(C) / (ms16 * 1e-3) / 1e9 / peak, 4)
        except Exception as e:  # e.g. a forced kernel variant without that mode
            detail['fprop'][str(C)]['acc_float16_ms'] = f'{type(e).__name__}'
            _lib.load().kdw_last_error()
    detail['clone'] = clone

    def roof(kind):
        """All launches of one operator in the timed region (one per C)."""
        ms, nbytes = tot[kind]
        ach = nbytes / (ms * 1e-3) / 1e9
        return {'bound': 'hbm', 'kernel': f'{kind}, all C', 'achieved': round(ach, 1), 'peak': peak,
                'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': round(ach / peak, 4), 'traffic': None,
                'avg_launch_ms': round(ms / len(channels), 4)}

    # the single kernel launch with the largest share of a step
    dom_kind, dom_C = max(((k, C) for k in ('fprop', 'wgrad') for C in channels),
                          key=lambda kc: detail[kc[0]][str(kc[1])]['ms'])
    dom = detail[dom_kind][str(dom_C)]
    full_size = SHAPE[0] == 350
    roofline = {'bound': 'hbm', 'kernel': f'{dom_kind} pass-1 kernel at C={dom_C}', 'achieved': dom['gbs'], 'peak': peak,
                'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': dom['frac'],
                'traffic': NCU_TRAFFIC.get((dom_kind, dom_C)) if full_size else None,
                'algorithmic_bytes': algorithmic_bytes(dom_C), 'avg_launch_ms': dom['ms']}
    step_bytes = sum(2 * algorithmic_bytes(C) for C in channels) * world
    value = step_bytes * args.steps / (total_ms * 1e-3) / 1e9

    e2e = measure_e2e(args, channels, dev, world, rank)
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = time_cpu_arm(channels, steps=2, warmup=1, min_seconds=8.0)
        cpu_baseline = {'value': round(sum(2 * algorithmic_bytes(C) for C in channels) / r['sec_per_step'] / 1e9, 3),
                        'unit': 'GB/s', 'cores': r['cores'], 'kind': 'port', 'sample': cpu_sample_text(r, channels)}
    triton_ref = triton_ops = None
    if args.compare_triton and rank == 0 and world == 1:
        triton_ref, triton_ops = measure_triton_reference(channels, data, dev)
    if rank == 0 and world == 1 and not args.no_small:
        detail['small_shape_latency'] = small_shape_latency(dev, triton_ops)

    line = None
    if rank == 0:
        line = {
            'metric': METRIC, 'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': round(total_ms / args.steps, 4), 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
            'config': sweep_config(channels, world), 'allreduce': reducer_name(reducer, world),
            'roofline': roofline, 'roofline_fprop': roof('fprop'), 'roofline_wgrad': roof('wgrad'),
            'cpu_baseline': cpu_baseline, 'e2e': e2e, 'clocks': clocks,
            'gpu_launches': (3 * len(channels) + (1 if reducer is not None else 0)) * args.steps, 'detail': detail,
            'device_status': status,
        }
        if triton_ref is not None:
            line['reference_triton_on_this_gpu'] = triton_ref
            try:  # how many times faster than the reference's own kernels on this GPU, per C
                line['vs_reference_triton'] = {
                    kind: {str(C): round(triton_ref[kind][str(C)]['ms'] / detail[kind][str(C)]['ms'], 2) for C in channels}
                    for kind in ('fprop', 'wgrad')}
            except (KeyError, TypeError):
                pass
    return line


def run_ours(args):
    import gc

    import torch

    ctx = Ctx(args)
    line = sweep_record(args, ctx)
    if not args.no_sharded and SHAPE[0] == 350:
        for name, fn in (('dshard', dshard_record), ('dpstep', dpstep_record)):
            gc.collect()
            torch.cuda.empty_cache()
            try:
                rec = fn(args, ctx, args.sub_steps, max(3, args.sub_warmup))
            except Exception as e:  # e.g. device memory: report it instead of losing the headline
                rec = {'error': f'{type(e).__name__}: {e}'[:300]}
            if line is not None:
                line[name] = rec
        if ctx.world == 1 and not args.no_fused:  # the two fused neighbours of the path, one GPU only
            gc.collect()
            torch.cuda.empty_cache()
            try:
                line['fused'] = fused_record(args, args.sub_steps)
            except Exception as e:
                line['fused'] = {'error': f'{type(e).__name__}: {e}'[:300]}
    if line is not None:
        print(json.dumps(line), flush=True)
    ctx.close()


def measure_e2e(args, channels, dev, world, rank):
    """The same sweep through the host-buffer operators: pinned host inputs, host outputs."""
    import torch
    import torch.distributed as dist

    from kerops_b200.host import DWConvHost, DWConvStepHost, DWConvWGRADHost

    if args.no_e2e:
        return None
    Cmax = max(channels)
    H, W, D = SHAPE
    # every rank pins three buffers of the largest volume; skip (and say so) rather than exhaust the host
    need = 3 * VOX * Cmax * 2 * world
    try:
        import psutil

        avail = psutil.virtual_memory().available
    except Exception:
        avail = None
    if avail is not None and need * 1.3 > avail:
        return {'value': None, 'unit': 'GB/s', 'skipped': f'pinned host buffers need {need >> 30} GiB over all ranks, '
                                                            f'{avail >> 30} GiB of host memory available'}
    # one pinned pool, sliced per C (contents: N(0,1) generated on the device once)
    pool = [torch.empty(VOX * Cmax, dtype=torch.float16, pin_memory=True) for _ in range(3)]
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    for p in pool[:2]:
        p.copy_(torch.randn(VOX * Cmax, generator=g, device=dev, dtype=torch.float16))
    torch.cuda.synchronize()

    def view(p, C):
        return p[:VOX * C].view(1, H, W, D, C).permute(0, 4, 1, 2, 3)

    wts = {C: ((torch.rand(3, 3, 3, C) * 2 - 1) / math.sqrt(27)).to(torch.float16).pin_memory() for C in channels}

    fused = args.e2e_api == 'step'

    def step():
        for C in channels:
            if fused:  # x crosses the bus once and feeds both kernels
                DWConvStepHost(view(pool[0], C), wts[C], view(pool[1], C), out=view(pool[2], C), device=dev)
            else:
                DWConvHost(view(pool[0], C), wts[C], out=view(pool[2], C), device=dev)
                DWConvWGRADHost(view(pool[0], C), view(pool[1], C), device=dev)

    n = max(1, min(args.steps, 3))
    step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(n):
        step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    # split calls: x for fprop, x and grad for wgrad; fused step: x and grad once; plus the weights
    h2d = sum((2 if fused else 3) * 2 * VOX * C + 54 * C for C in channels)
    d2h = sum(2 * VOX * C + 54 * C for C in channels)      # y; dw
    nbytes = sum(2 * algorithmic_bytes(C) for C in channels) * world
    return {'value': round(nbytes * n / dt / 1e9, 2), 'unit': 'GB/s', 'h2d_bytes_per_step': h2d,
            'd2h_bytes_per_step': d2h, 'steps': n, 'ms_per_step': round(dt / n * 1e3, 2),
            'api': ('kerops_b200.host.DWConvStepHost (forward + weight gradient of one host volume per call'
                    if fused else 'kerops_b200.host.DWConvHost then DWConvWGRADHost (two calls per volume')
                   + '; pinned host buffers, slab pipeline)'}


def measure_triton_reference(channels, data, dev):
    """Optional comparator: the unmodified reference Triton kernels (installed under baseline/_ref) on this GPU."""
    import torch

    ref_root = os.path.join(ROOT, 'baseline', '_ref')
    if not os.path.isdir(os.path.join(ref_root, 'kerops')):
        return {'unavailable': 'baseline/_ref/kerops not present'}, None
    sys.path.insert(0, ref_root)
    try:
        from kerops.ops.conv import DWConv as RefDWConv, DWConvWGRAD as RefDWConvWGRAD
    except Exception as e:
        return {'unavailable': f'{type(e).__name__}: {e}'}, None
    out = {'fprop': {}, 'wgrad': {}}
    for C in channels:
        x, grad, w = data[C]
        for name, fn in (('fprop', lambda: RefDWConv(x, w)), ('wgrad', lambda: RefDWConvWGRAD(x, grad))):
            try:
                for _ in range(3):
                    fn()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / 5
                out[name][str(C)] = {'ms': round(ms, 4), 'gbs': round(algorithmic_bytes(C) / (ms * 1e-3) / 1e9, 1)}
            except Exception as e:
                out[name][str(C)] = {'error': f'{type(e).__name__}: {e}'[:200]}
    return out, (RefDWConv, RefDWConvWGRAD)


def dshard_record(args, ctx, steps, warmup):
    """configs[3]: one (1, 128, 1400, 350, 128) volume sharded along H over the ranks (1-plane halos exchanged
    point to point, fp32 weight gradient all-reduced); strong scaling.  A step = forward + weight gradient.
    Returns the record (on every rank)."""
    import torch

    from kerops_b200 import _lib
    from kerops_b200 import dist as kd

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    C, H, W, D = 128, args.dshard_planes, SHAPE[1], SHAPE[2]
    hb, he = kd.shard_planes(H, world, rank)
    Hs = he - hb
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    xh = kd.alloc_halo_volume(1, C, Hs, W, D, dev)
    xh[:, :, 1:-1].copy_(torch.randn(1, Hs, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3))
    grad = torch.randn(1, Hs, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device=dev) * 2 - 1) / math.sqrt(27)).to(torch.float16)
    y = torch.empty((1, Hs, W, D, C), dtype=torch.float16, device=dev).permute(0, 4, 1, 2, 3)
    reducer = make_reducer(args, 27 * C, world)
    names = ['fprop_interior', 'halo_wait', 'fprop_boundary', 'wgrad', 'allreduce']

    def step(events=None):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] if events is not None else None
        kd.hsharded_step(xh, w, grad, y=y, reducer=reducer, events=ev)
        if events is not None:
            events.append(ev)

    sampler = ClockSampler(dev)
    sampler.start()
    for _ in range(warmup):
        step()
    ctx.barrier()
    sampler.begin()
    events = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step(events)
    e1.record()
    ctx.barrier()
    clocks = sampler.stop()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    parts = breakdown(ctx, names, events)
    status = _lib.device_status()
    peak, peak_kind = measured_peak()
    nbytes = 2 * 4 * H * W * D * C  # forward + weight gradient over the whole volume
    value = nbytes * steps / (ms * 1e-3) / 1e9
    return {
        'metric': 'DWConv + DWConvWGRAD algorithmic HBM GB/s on one H-sharded (1,128,%d,350,128) fp16 volume' % H,
        'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': round(ms / steps, 4), 'higher_is_better': True, 'scaling': 'strong',
        'workload': f'configs[3]: (1,128,{H},350,128) split along H over {world} rank(s), 1-plane halos over NCCL '
                    'point-to-point overlapped with the interior planes, fp32 [27][128] gradient all-reduced',
        'allreduce': reducer_name(reducer, world), 'per_gpu_frac_of_peak': round(value / world / peak, 4),
        'peak': peak, 'peak_kind': peak_kind, 'breakdown_ms_per_rank': parts,
        'gpu_launches_per_step': (5 if world > 1 else 3) + (1 if reducer is not None else 0),
        'clocks': clocks, 'device_status': status,
    }


def dpstep_record(args, ctx, steps, warmup):
    """configs[4]: data-parallel slice of a training step.  A batch of 8 samples (32, 350, 350, 128) is split by
    sample over the ranks (8, 4, 2, 1 samples per rank on 1, 2, 4, 8 GPUs); a step is DWConv of the local samples,
    DWConvWGRAD against an N(0,1) gradient, and one all-reduce of the fp32 [27][32] weight gradient.  Strong
    scaling: the batch is fixed."""
    import torch

    from kerops_b200 import _lib
    from kerops_b200 import dist as kd

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    batch, C = args.dp_batch, 32
    H, W, D = SHAPE
    if batch % world:
        raise SystemExit(f'--dp-batch {batch} is not a multiple of the {world} ranks')
    n_local = batch // world
    xs, gs = [], []
    for i in range(n_local):  # one seed per global sample index, so any sharding sees the same batch
        g = torch.Generator(device=dev).manual_seed(9000 + rank * n_local + i)
        xs.append(torch.randn(1, H, W, D, C, generator=g, device=dev, dtype=torch.float16))
        gs.append(torch.randn(1, H, W, D, C, generator=g, device=dev, dtype=torch.float16))
    x = torch.cat(xs).permute(0, 4, 1, 2, 3)
    grad = torch.cat(gs).permute(0, 4, 1, 2, 3)
    del xs, gs
    gw = torch.Generator(device=dev).manual_seed(77)
    w = ((torch.rand(3, 3, 3, C, generator=gw, device=dev) * 2 - 1) / math.sqrt(27)).to(torch.float16)
    y = torch.empty((n_local, H, W, D, C), dtype=torch.float16, device=dev).permute(0, 4, 1, 2, 3)
    reducer = make_reducer(args, 27 * C, world)
    names = ['fprop', 'wgrad', 'allreduce']

    def step(events=None):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] if events is not None else None
        kd.sample_sharded_step(x, w, grad, reducer=reducer, y=y, events=ev)
        if events is not None:
            events.append(ev)

    sampler = ClockSampler(dev)
    sampler.start()
    for _ in range(warmup):
        step()
    ctx.barrier()
    sampler.begin()
    events = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step(events)
    e1.record()
    ctx.barrier()
    clocks = sampler.stop()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    parts = breakdown(ctx, names, events)
    status = _lib.device_status()
    peak, peak_kind = measured_peak()
    nbytes = 2 * algorithmic_bytes(C, batch)
    value = nbytes * steps / (ms * 1e-3) / 1e9
    return {
        'metric': 'DWConv + DWConvWGRAD algorithmic HBM GB/s, batch of %d (32,%d,350,128) fp16 samples' % (batch, H),
        'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': round(ms / steps, 4), 'higher_is_better': True, 'scaling': 'strong',
        'workload': f'configs[4]: batch {batch} x (32,{H},350,128), {n_local} sample(s) per rank; DWConv, DWConvWGRAD, '
                    'all-reduce of the fp32 [27][32] gradient',
        'allreduce': reducer_name(reducer, world), 'per_gpu_frac_of_peak': round(value / world / peak, 4),
        'peak': peak, 'peak_kind': peak_kind, 'breakdown_ms_per_rank': parts,
        'gpu_launches_per_step': 3 + (1 if reducer is not None else 0),
        'clocks': clocks, 'device_status': status,
    }


def run_sharded(args, fn):
    """--workload dshard / dpstep alone: the record as the JSON line."""
    ctx = Ctx(args)
    rec = fn(args, ctx, args.steps, args.warmup)
    if ctx.rank == 0:
        rec.update({'vs_baseline': None, 'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
                    'config': {'workload': rec['workload'], 'l2': 'inputs larger than L2',
                               'parallelism': ('hshard' if fn is dshard_record else 'dp') + str(ctx.world)},
                    'roofline': {'bound': 'hbm', 'kernel': 'fprop + wgrad, whole step',
                                 'achieved': round(rec['value'] / ctx.world, 1), 'peak': rec['peak'],
                                 'peak_kind': rec['peak_kind'], 'unit': 'GB/s', 'frac': rec['per_gpu_frac_of_peak'],
                                 'traffic': None},
                    'gpu_launches': rec['gpu_launches_per_step'] * rec['steps']})
        print(json.dumps(rec), flush=True)
    ctx.close()


def run_fused(args):
    """--workload fused alone: the record as the JSON line."""
    print(json.dumps(fused_record(args, args.steps)), flush=True)


def fused_record(args, steps):
    """The fused neighbours, per C of the sweep, one GPU.  Headline: DWConvAddStats(x, weight, residual), algorithmic
    bytes per call read x + read residual + write out = 6*V*C; comparators timed in the same run: our DWConv followed
    by a torch fp16 add and channel means, and - when baseline/_ref is present - the reference's
    AddStats(DWConv(...)).  Also timed (detail[C]['bnrelu']): DWConvBNReLU against the reference's
    DWConv(ApplyBNReLU(...))."""
    import torch

    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConv, DWConvAddStats, DWConvBNReLU

    dev = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    torch.cuda.set_device(dev)
    _lib.load()
    peak, peak_kind = measured_peak()
    ref_ops = None
    ref_root = os.path.join(ROOT, 'baseline', '_ref')
    if args.compare_triton and os.path.isdir(os.path.join(ref_root, 'kerops')):
        sys.path.append(ref_root)
        try:
            from kerops.ops.addition import AddStats as RefAddStats
            from kerops.ops.bnrelu import ApplyBNReLU as RefApplyBNReLU
            from kerops.ops.conv import DWConv as RefDWConv

            ref_ops = (RefDWConv, RefAddStats, RefApplyBNReLU)
        except Exception:
            ref_ops = None

    def timeit(fn, reps):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def unfused(x, w, r):
        out = DWConv(x, w) + r
        o = out.float()
        return out, o.mean(dim=(0, 2, 3, 4)), (o * o).mean(dim=(0, 2, 3, 4))

    detail, tot_ms, tot_bytes = {}, 0.0, 0
    sampler = ClockSampler(dev)
    sampler.start()
    sampler.begin()
    for C in args.channels:
        x, r, w = make_gpu_inputs(C, dev, seed=C)
        nbytes = 6 * VOX * C
        ms = timeit(lambda: DWConvAddStats(x, w, r), steps)
        row = {'ms': round(ms, 4), 'gbs': round(nbytes / ms / 1e6, 1), 'frac': round(nbytes / ms / 1e6 / peak, 4),
               'unfused_ms': round(timeit(lambda: unfused(x, w, r), 3), 4)}
        if ref_ops is not None:
            try:
                row['reference_chain_ms'] = round(timeit(lambda: ref_ops[1](ref_ops[0](x, w), r), 3), 4)
            except Exception as e:
                row['reference_chain_ms'] = f'{type(e).__name__}'
        # the prologue neighbour: y = DWConv(relu(x * scale + shift)); algorithmic bytes 4*V*C like the plain conv
        scale, shift = torch.rand(C, device=dev) + 0.5, torch.randn(C, device=dev) * 0.5
        ms_b = timeit(lambda: DWConvBNReLU(x, scale, shift, w), steps)
        ms_h = timeit(lambda: DWConvBNReLU(x, scale, shift, w, PROLOGUE='float16'), steps)
        row['bnrelu'] = {'ms': round(ms_b, 4), 'gbs': round(4 * VOX * C / ms_b / 1e6, 1),
                         'frac': round(4 * VOX * C / ms_b / 1e6 / peak, 4), 'ms_packed_half_prologue': round(ms_h, 4)}
        if ref_ops is not None:
            try:
                row['bnrelu']['reference_chain_ms'] = round(
                    timeit(lambda: ref_ops[0](ref_ops[2](x, scale, shift), w), 3), 4)
            except Exception as e:
                row['bnrelu']['reference_chain_ms'] = f'{type(e).__name__}'
        detail[str(C)] = row
        tot_ms += ms
        tot_bytes += nbytes
        del x, r, w
    clocks = sampler.stop()
    value = tot_bytes / tot_ms / 1e6
    return {
        'metric': 'DWConvAddStats algorithmic HBM GB/s at (1,C,%d,350,128) fp16 channels_last_3d' % SHAPE[0],
        'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': 1, 'steps': steps, 'warmup': 3,
        'ms_per_step': round(tot_ms, 4), 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
        'config': {'workload': 'fused forward + residual add + channel statistics, C in '
                               + ','.join(map(str, args.channels)), 'l2': 'inputs larger than L2'},
        'roofline': {'bound': 'hbm', 'kernel': 'fprop_addstats_kernel, all C', 'achieved': round(value, 1), 'peak': peak,
                     'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': round(value / peak, 4), 'traffic': None},
        'clocks': clocks, 'gpu_launches': 4 * len(args.channels) * steps, 'detail': detail,
        'device_status': _lib.device_status(),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--channels', default=','.join(map(str, ALL_CHANNELS)))
    ap.add_argument('--planes', type=int, default=SHAPE[0],
                    help='h extent of the volume (default 350); smaller values are for profiler captures only')
    ap.add_argument('--no-fused', action='store_true', help='sweep workload at one GPU: skip the `fused` sub-record')
    ap.add_argument('--workload', default='sweep', choices=['sweep', 'dshard', 'dpstep', 'fused'],
                    help="'sweep' (default): the headline per-C sweep, one sample per GPU; 'dshard': one large volume "
                         "sharded along H over the GPUs; 'dpstep': a batch of (32,350,350,128) samples split by sample; 'fused': DWConvAddStats, one GPU")
    ap.add_argument('--dp-batch', type=int, default=8)
    ap.add_argument('--allreduce', default='push', choices=['nccl', 'push'],
                    help="how the fp32 weight gradients are summed over the ranks: NCCL, or the library's own "
                         'push/flag/sum kernel over peer memory')
    ap.add_argument('--dshard-planes', type=int, default=1400)
    ap.add_argument('--no-sharded', action='store_true',
                    help='sweep workload: skip the dshard / dpstep sub-records')
    ap.add_argument('--sub-steps', type=int, default=5, help='timed steps of the dshard / dpstep sub-records')
    ap.add_argument('--sub-warmup', type=int, default=3)
    ap.add_argument('--no-small', action='store_true', help='skip the small-shape latency measurement')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--e2e-api', default='step', choices=['step', 'split'],
                    help="'step': one DWConvStepHost call per volume (x is copied once); 'split': DWConvHost and "
                         'DWConvWGRADHost as two calls')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--compare-triton', dest='compare_triton', action='store_true', default=True,
                    help='also time the reference Triton kernels from baseline/_ref on this GPU (default at 1 GPU; '
                         'reported as reference_triton_on_this_gpu, or why it is unavailable)')
    ap.add_argument('--no-compare-triton', dest='compare_triton', action='store_false')
    args = ap.parse_args()
    args.channels = [int(c) for c in args.channels.split(',')]
    set_planes(args.planes)
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup
    if args.impl == 'reference':
        run_reference(args)
    elif args.workload == 'dshard':
        run_sharded(args, dshard_record)
    elif args.workload == 'dpstep':
        run_sharded(args, dpstep_record)
    elif args.workload == 'fused':
        run_fused(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
