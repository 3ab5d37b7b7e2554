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
fraction, ratio to torch.clone), `e2e` (the same sweep through the host-buffer operator DWConvStepHost,
host<->device copies inside the timed region), `cpu_baseline` (torch CPU depthwise conv3d, the check the
reference's tests use, on a bounded sample), `clocks` (SM clock and throttle reasons sampled through NVML during
the timed region), and at one GPU `reference_triton_on_this_gpu` (the reference's own Triton kernels from
baseline/_ref timed on the same tensors).

Other workloads (--workload): `dshard` = one (1,128,1400,350,128) volume sharded along H over the ranks with halo
exchange (strong scaling); `dpstep` = a batch of 8 x (32,350,350,128) samples split by sample (strong scaling);
`fused` = DWConvAddStats and DWConvBNReLU against the unfused and the reference two-operator chains (one GPU).

`--impl reference` times the CPU arm alone (rank 0 only): torch conv3d(groups=C) forward + weight
gradient on the host cores, one (1, 8, 350, 350, 128) volume per step.
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu capture summarised in
# profiles/fprop_wgrad_c8_c32_c128_planes100.md: captured on (1, C, 100, 350, 128) volumes and scaled by
# 350/100 planes (traffic grows in proportion to the planes a launch processes).  Bytes per (1,C,350,350,128)
# launch; None where no capture has been taken.
NCU_TRAFFIC = {
    ('fprop', 8): int((0.078799 + 0.026727) * 3.5e9),
    ('wgrad', 8): int((0.156367 + 0.004412) * 3.5e9),
    ('fprop', 32): int((0.290660 + 0.248650) * 3.5e9),
    ('wgrad', 32): int((0.581526 + 0.006321) * 3.5e9),
    ('fprop', 128): int((1.344124 + 1.114130) * 3.5e9),
    ('wgrad', 128): int((2.334769 + 0.006344) * 3.5e9),
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
def make_cpu_inputs(C, seed=0):
    import torch

    g = torch.Generator().manual_seed(seed)
    H, W, D = SHAPE
    x = torch.randn(1, H, W, D, C, generator=g, dtype=torch.float32).to(torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(1, H, W, D, C, generator=g, dtype=torch.float32).to(torch.float16).permute(0, 4, 1, 2, 3)
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


def time_cpu_arm(C, steps, warmup, min_seconds=0.0):
    """Seconds per step (median) of the faster of the fp32 / fp16 torch CPU paths, its name, the CPU seconds spent
    in its timed steps and their number.  At least `steps` steps, and more until `min_seconds` of work are done."""
    import torch

    x, grad, w = make_cpu_inputs(C)
    best = None
    for dtype in (torch.float32, torch.float16):
        try:
            for _ in range(warmup):
                cpu_step(x, grad, w, dtype)
            ts = []
            while len(ts) < steps or (sum(ts) < min_seconds and len(ts) < 500):
                t0 = time.perf_counter()
                cpu_step(x, grad, w, dtype)
                ts.append(time.perf_counter() - t0)
            med = statistics.median(ts)
            if best is None or med < best[0]:
                best = (med, str(dtype).replace('torch.', ''), sum(ts), len(ts))
        except Exception:
            continue
    if best is None:
        raise RuntimeError('torch CPU conv3d failed in both fp32 and fp16')
    return best


def run_reference(args):
    import torch

    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    C = 8
    cores = torch.get_num_threads()
    med, dtype, _, _ = time_cpu_arm(C, args.steps, max(1, args.warmup))
    nbytes = 2 * algorithmic_bytes(C)
    value = nbytes / med / 1e9
    sample = f'one (1,{C},350,350,128) volume per step: conv3d(groups=C) forward + weight gradient, torch CPU {dtype}'
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': 'GB/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': med * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': dtype, 'data': 'synthetic',
        'config': {'workload': f'DWConv + DWConvWGRAD on (1,{C},350,350,128) fp16 channels_last_3d, host cores'},
        'cpu_baseline': {'value': value, 'unit': 'GB/s', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': 'GB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
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


def run_ours(args):
    import torch
    import torch.distributed as dist

    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConv, _launch

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus and world > 1:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}')
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: kerops_b200 has no CPU path')
    dev = torch.device('cuda', local)
    torch.cuda.set_device(dev)
    _lib.load()
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)

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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(dev)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.begin()
    events = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        step(events)
    t_end.record()
    barrier()
    clocks = sampler.stop()
    total_ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
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
    # torch.clone of the same tensors, the comparator the reference's README uses
    clone = {}
    for C in channels:
        x = data[C][0]
        for _ in range(2):
            x.clone()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            x.clone()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 5
        clone[str(C)] = {'ms': round(ms, 4), 'gbs': round(algorithmic_bytes(C) / (ms * 1e-3) / 1e9, 1)}
        for kind in ('fprop', 'wgrad'):
            detail[kind][str(C)]['x_clone'] = round(detail[kind][str(C)]['ms'] / ms, 3)
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
    roofline = {'bound': 'hbm', 'kernel': f'{dom_kind}_tma_kernel at C={dom_C}', 'achieved': dom['gbs'], 'peak': peak,
                'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': dom['frac'],
                'traffic': NCU_TRAFFIC.get((dom_kind, dom_C)) if full_size else None,
                'algorithmic_bytes': algorithmic_bytes(dom_C), 'avg_launch_ms': dom['ms']}
    step_bytes = sum(2 * algorithmic_bytes(C) for C in channels) * world
    value = step_bytes * args.steps / (total_ms * 1e-3) / 1e9

    e2e = measure_e2e(args, channels, dev, world, rank)
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = torch.get_num_threads()
        med, dtype, spent, n_cpu = time_cpu_arm(8, steps=2, warmup=1, min_seconds=8.0)
        cpu_baseline = {
            'value': round(2 * algorithmic_bytes(8) / med / 1e9, 3), 'unit': 'GB/s', 'cores': cores, 'kind': 'port',
            'sample': f'(1,8,350,350,128) only: torch CPU conv3d(groups=8) forward + weight gradient in {dtype}, '
                      f'median of {n_cpu} steps after 1 warm-up ({spent:.1f} s of CPU work)',
        }
    triton_ref = measure_triton_reference(channels, data, dev) if (args.compare_triton and rank == 0 and world == 1) else None

    if rank == 0:
        line = {
            'metric': METRIC, 'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': round(total_ms / args.steps, 4), 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
            'config': {
                'workload': f'configs[1]+[2]: DWConv then DWConvWGRAD on (1,C,{SHAPE[0]},350,128) fp16 channels_last_3d for C in '
                            + ','.join(map(str, channels)) + '; one sample per GPU',
                'l2': 'inputs larger than L2 (smallest tensor 251 MB; 31 GB touched per step)',
                'parallelism': f'dp{world}' if world > 1 else 'single',
                'allreduce': ('push kernel over peer memory' if reducer is not None else 'nccl') if world > 1 else None,
            },
            'roofline': roofline, 'roofline_fprop': roof('fprop'), 'roofline_wgrad': roof('wgrad'),
            'cpu_baseline': cpu_baseline, 'e2e': e2e, 'clocks': clocks,
            'gpu_launches': (3 * len(channels) + (1 if reducer is not None else 0)) * args.steps, 'detail': detail, 'device_status': status,
        }
        if triton_ref is not None:
            line['reference_triton_on_this_gpu'] = triton_ref
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
        return {'unavailable': 'baseline/_ref/kerops not present'}
    sys.path.insert(0, ref_root)
    try:
        from kerops.ops.conv import DWConv as RefDWConv, DWConvWGRAD as RefDWConvWGRAD
    except Exception as e:
        return {'unavailable': f'{type(e).__name__}: {e}'}
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
    return out


def run_dshard(args):
    """configs[3]: one (1, 128, 1400, 350, 128) volume sharded along H over the ranks (1-plane halos exchanged
    point to point, fp32 weight gradient all-reduced); strong scaling.  A step = forward + weight gradient."""
    import torch
    import torch.distributed as dist

    from kerops_b200 import _lib
    from kerops_b200 import dist as kd

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    dev = torch.device('cuda', local)
    torch.cuda.set_device(dev)
    _lib.load()
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    C, H, W, D = 128, args.dshard_planes, SHAPE[1], SHAPE[2]
    hb, he = kd.shard_planes(H, world, rank)
    Hs = he - hb
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    xh = kd.alloc_halo_volume(1, C, Hs, W, D, dev)
    xh[:, :, 1:-1].copy_(torch.randn(1, Hs, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3))
    grad = torch.randn(1, Hs, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device=dev) * 2 - 1) / math.sqrt(27)).to(torch.float16)

    reducer = make_reducer(args, 27 * C, world)

    class Single:  # one rank: no neighbours, the halo planes stay zero
        @staticmethod
        def finish():
            return None

    def step():
        if world > 1:
            fin = kd.exchange_halo(xh)
            y = kd.hsharded_fprop(xh, w, halo_ready=fin)
            dw = kd.hsharded_wgrad(xh, grad, halo_ready=lambda: None, reducer=reducer)  # halo already in place
        else:
            y = kd.hsharded_fprop(xh, w, halo_ready=Single.finish)
            dw = kd.hsharded_wgrad(xh, grad, halo_ready=Single.finish, reduce=False)
        return y, dw

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(dev)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    status = _lib.device_status()
    peak, peak_kind = measured_peak()
    nbytes = 2 * 4 * H * W * D * C  # forward + weight gradient over the whole volume
    value = nbytes * args.steps / (ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            'metric': 'DWConv + DWConvWGRAD algorithmic HBM GB/s on one H-sharded (1,128,%d,350,128) fp16 volume' % H,
            'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': round(ms / args.steps, 4), 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
            'config': {'workload': f'configs[3]: (1,128,{H},350,128) split along H over {world} rank(s), 1-plane halos '
                                   'over NCCL point-to-point, fp32 [27][128] gradient all-reduced ('
                                   + ('push kernel over peer memory' if reducer is not None else 'nccl') + ')',
                       'l2': 'inputs larger than L2', 'parallelism': f'hshard{world}'},
            'roofline': {'bound': 'hbm', 'kernel': 'fprop + wgrad, whole step', 'achieved': round(value / world, 1),
                         'peak': peak, 'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': round(value / world / peak, 4),
                         'traffic': None},
            'clocks': clocks, 'gpu_launches': ((9 if world > 1 else 3) + (1 if reducer is not None else 0)) * args.steps,
            'device_status': status,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_dpstep(args):
    """configs[4]: data-parallel slice of a training step.  A batch of 8 samples (32, 350, 350, 128) is split by
    sample over the ranks (8, 4, 2, 1 samples per rank on 1, 2, 4, 8 GPUs); a step is DWConv of the local samples,
    DWConvWGRAD against an N(0,1) gradient, and one all-reduce of the fp32 [27][32] weight gradient.  Strong
    scaling: the batch is fixed."""
    import torch
    import torch.distributed as dist

    from kerops_b200 import _lib
    from kerops_b200 import dist as kd

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    dev = torch.device('cuda', local)
    torch.cuda.set_device(dev)
    _lib.load()
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    reducer = make_reducer(args, 27 * C, world)
    sampler = ClockSampler(dev)
    sampler.start()
    for _ in range(args.warmup):
        kd.sample_sharded_step(x, w, grad, reducer=reducer)
    barrier()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        kd.sample_sharded_step(x, w, grad, reducer=reducer)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    status = _lib.device_status()
    peak, peak_kind = measured_peak()
    nbytes = 2 * algorithmic_bytes(C, batch)
    value = nbytes * args.steps / (ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            'metric': 'DWConv + DWConvWGRAD algorithmic HBM GB/s, batch of %d (32,%d,350,128) fp16 samples' % (batch, H),
            'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': round(ms / args.steps, 4), 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
            'config': {'workload': f'configs[4]: batch {batch} x (32,{H},350,128), {n_local} sample(s) per rank; DWConv, '
                                   'DWConvWGRAD, all-reduce of the fp32 [27][32] gradient ('
                                   + ('push kernel over peer memory' if reducer is not None else 'nccl') + ')',
                       'l2': 'inputs larger than L2', 'parallelism': f'dp{world}'},
            'roofline': {'bound': 'hbm', 'kernel': 'fprop + wgrad, whole step', 'achieved': round(value / world, 1),
                         'peak': peak, 'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': round(value / world / peak, 4),
                         'traffic': None},
            'clocks': clocks, 'gpu_launches': (3 + (1 if reducer is not None else 0)) * args.steps,
            'device_status': status,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_fused(args):
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
        ms = timeit(lambda: DWConvAddStats(x, w, r), args.steps)
        row = {'ms': round(ms, 4), 'gbs': round(nbytes / ms / 1e6, 1), 'frac': round(nbytes / ms / 1e6 / peak, 4),
               'unfused_ms': round(timeit(lambda: unfused(x, w, r), 3), 4)}
        if ref_ops is not None:
            try:
                row['reference_chain_ms'] = round(timeit(lambda: ref_ops[1](ref_ops[0](x, w), r), 3), 4)
            except Exception as e:
                row['reference_chain_ms'] = f'{type(e).__name__}'
        # the prologue neighbour: y = DWConv(relu(x * scale + shift)); algorithmic bytes 4*V*C like the plain conv
        scale, shift = torch.rand(C, device=dev) + 0.5, torch.randn(C, device=dev) * 0.5
        ms_b = timeit(lambda: DWConvBNReLU(x, scale, shift, w), args.steps)
        ms_h = timeit(lambda: DWConvBNReLU(x, scale, shift, w, PROLOGUE='float16'), args.steps)
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
    print(json.dumps({
        'metric': 'DWConvAddStats algorithmic HBM GB/s at (1,C,%d,350,128) fp16 channels_last_3d' % SHAPE[0],
        'value': round(value, 1), 'unit': 'GB/s', 'n_gpus': 1, 'steps': args.steps, 'warmup': 3,
        'ms_per_step': round(tot_ms, 4), 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'f16 products, f32 accumulation', 'data': 'synthetic',
        'config': {'workload': 'fused forward + residual add + channel statistics, C in '
                               + ','.join(map(str, args.channels)), 'l2': 'inputs larger than L2'},
        'roofline': {'bound': 'hbm', 'kernel': 'fprop_addstats_kernel, all C', 'achieved': round(value, 1), 'peak': peak,
                     'peak_kind': peak_kind, 'unit': 'GB/s', 'frac': round(value / peak, 4), 'traffic': None},
        'clocks': clocks, 'gpu_launches': 4 * len(args.channels) * args.steps, 'detail': detail,
        'device_status': _lib.device_status(),
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--channels', default=','.join(map(str, ALL_CHANNELS)))
    ap.add_argument('--planes', type=int, default=SHAPE[0],
                    help='h extent of the volume (default 350); smaller values are for profiler captures only')
    ap.add_argument('--workload', default='sweep', choices=['sweep', 'dshard', 'dpstep', 'fused'],
                    help="'sweep' (default): the headline per-C sweep, one sample per GPU; 'dshard': one large volume "
                         "sharded along H over the GPUs; 'dpstep': a batch of (32,350,350,128) samples split by sample; 'fused': DWConvAddStats, one GPU")
    ap.add_argument('--dp-batch', type=int, default=8)
    ap.add_argument('--allreduce', default='push', choices=['nccl', 'push'],
                    help="how the fp32 weight gradients are summed over the ranks: NCCL, or the library's own "
                         'push/flag/sum kernel over peer memory')
    ap.add_argument('--dshard-planes', type=int, default=1400)
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
        run_dshard(args)
    elif args.workload == 'dpstep':
        run_dpstep(args)
    elif args.workload == 'fused':
        run_fused(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
