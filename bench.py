"""Benchmark of the WKV7 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: WKV7 forward+backward at the 124M shape (B=64 per GPU, T=1024, H=12, N=64, bf16 inputs,
fp32 state), seeded synthetic inputs with the value distributions of the workload definition.  A
step is one forward and one backward over the device-resident batch.  With N > 1 (launched under
torchrun, one rank per GPU) every rank processes its own batch shard; chains are independent, so
there is no collective on the data path ("weak" scaling) and NCCL is used only to take the maximum
time over ranks.  One JSON line is printed by rank 0.

`--workload attn_ln|prefill|ddlerp|expand_loras|mixer|proj` time the other workloads of the path (prefill also under
torchrun: config 4 with its 8 sequences sharded over the ranks, "strong" scaling); the default run reports them under
`secondary`.  `--impl reference-cuda` times the reference's own CUDA kernels from baseline/_ref (context only).

`--impl reference` times the reference's own CPU implementation of the path — the naive per-step
recurrence, restated in oracle/wkv7_ref.py, forward + autograd backward — on the host cores, on a
bounded batch slice of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, 'wind-rwkv7_b200')]

import torch as th  # noqa: E402

METRIC = 'WKV7 fwd+bwd Mtokens/s per GPU at H12 N64 T1024 bf16; % of HBM/TC roofline'
B_PER_GPU, T, H, N = 64, 1024, 12, 64
FWD_BYTES_PER_TOKEN_HEAD = 7 * N * 2    # r,w,k,v,a,b in + y out, bf16
BWD_BYTES_PER_TOKEN_HEAD = 13 * N * 2   # r,w,k,v,a,b,dy in + six gradients out, bf16
# Fallback copy of the pool's measured STREAM-style bandwidth, used when MEASURED_PEAKS.json is absent.
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch at this workload, from an ncu capture of
# `python bench.py --no-e2e --no-cpu-baseline --steps 1 --warmup 1 --batch 16`: 428.1 MB read + 130.8 MB written at
# B = 16, scaled by 4 (traffic is proportional to the number of chains; the B = 64 workload is too large to capture).
BWD_DRAM_TRAFFIC_BYTES = 2_235_450_000


def hbm_peak():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        return float(json.load(open(p))['hbm_gbs']), 'measured'
    return FALLBACK_HBM_GBS, 'fallback'


class ClockSampler:
    """Samples SM clock and throttle reasons (NVML) while the timed region runs."""

    def __init__(self, device):
        self.device, self.samples, self.stop, self.thread = device, [], False, None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            try:
                uuid = 'GPU-' + str(th.cuda.get_device_properties(self.device).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                h = nv.nvmlDeviceGetHandleByIndex(self.device)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            while not self.stop:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((mhz, reasons))
                time.sleep(0.002)
        except Exception as e:  # no NVML: report it rather than guess
            self.error = repr(e)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        time.sleep(0.05)
        self.samples.clear()
        return self

    def __exit__(self, *a):
        self.stop = True
        self.thread.join(timeout=10)

    def summary(self):
        if not self.samples:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['unsampled: ' + getattr(self, 'error', 'no samples')]}
        mhz = sorted(s[0] for s in self.samples)
        bits = {'hw_slowdown': 0x8, 'sw_power_cap': 0x4, 'sw_thermal_slowdown': 0x20, 'hw_thermal_slowdown': 0x40}
        reasons = [n for n, b in bits.items() if any(s[1] & b for s in self.samples)]
        return {'sm_mhz': mhz[len(mhz) // 2], 'sm_max_mhz': self.max_mhz, 'reasons': reasons, 'samples': len(mhz)}


def shard_of(rank, world, total):
    """Contiguous batch shard [lo, hi) of `total` items for `rank` (used by the sharded tests)."""
    per, rem = divmod(total, world)
    lo = rank * per + min(rank, rem)
    return lo, lo + per + (1 if rank < rem else 0)


def max_over_ranks(ms, dist, device):
    t = th.tensor([ms], dtype=th.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def cpu_reference_run(sample_B, steps, warmup):
    """The reference's CPU recurrence (restated in oracle/wkv7_ref.py) on a batch slice, fwd+bwd, on all host cores
    (torchrun exports OMP_NUM_THREADS=1 to its ranks; the thread count is set here explicitly)."""
    th.set_num_threads(max(1, os.cpu_count() or 1))
    sys.path.insert(0, os.path.join(ROOT, 'oracle'))
    import wkv7_ref
    from wind_rwkv.rwkv7 import synthetic
    d = synthetic.wkv7_inputs(sample_B, T, H, N, seed=1, dtype=th.bfloat16)
    ins = [d[n].requires_grad_() for n in 'rwkvab']
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        y = wkv7_ref.ref_attn(*ins, N)
        y.backward(d['dy'])
        for x in ins:
            x.grad = None
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return sample_B * T / sec / 1e6, sec


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    sample_B = 4
    val, sec = cpu_reference_run(sample_B, max(1, min(args.steps, 3)), 1 if args.warmup else 0)
    cores = th.get_num_threads()
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': 'Mtokens/s', 'n_gpus': args.gpus,
        'steps': max(1, min(args.steps, 3)), 'warmup': 1 if args.warmup else 0, 'ms_per_step': sec * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': f'WKV7 fwd+bwd B{B_PER_GPU} T{T} H{H} N{N} (bounded sample: B={sample_B} of {B_PER_GPU})',
                   'note': 'CPU arm: one process on the host cores of the box; its value does not depend on --gpus'},
        'cpu_baseline': {'value': val, 'unit': 'Mtokens/s', 'cores': cores, 'kind': 'port',
                         'sample': f'B={sample_B} of {B_PER_GPU}, T={T}, H={H}: torch fp32 per-step recurrence, '
                                   f'forward + autograd backward, {cores} threads'},
        'e2e': {'value': val, 'unit': 'Mtokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }
    print(json.dumps(line))


def bind_to_gpu_numa_node(device_index):
    """Restricts this process to the CPUs of the NUMA node its GPU is attached to, so that the pinned host buffers
    allocated afterwards (first touch) come from that node's memory.  Returns what was found and done."""
    info = {'numa_node': None, 'cpus': None}
    try:
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByUUID('GPU-' + str(th.cuda.get_device_properties(device_index).uuid))
        bus = nv.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(':')[0]) == 8:       # NVML prints an 8-digit PCI domain, sysfs a 4-digit one
            bus = bus[4:]
        node = int(open(f'/sys/bus/pci/devices/{bus}/numa_node').read())
        info['numa_node'] = node
        if node < 0:
            return info
        cpus = set()
        for part in open(f'/sys/devices/system/node/node{node}/cpulist').read().strip().split(','):
            lo, _, hi = part.partition('-')
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info['cpus'] = len(cpus)
    except Exception as e:  # no NVML / no sysfs entry: leave the affinity alone and say so
        info['error'] = repr(e)
    return info


def run_prefill(args):
    """Config 4 (B8 T65536 H40, s0 -> sT, forward only) with the batch sharded over the ranks: "strong" scaling,
    every rank runs B/N of the 8 sequences, no collective on the data path."""
    from wind_rwkv.rwkv7 import _lib, attn, synthetic
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    th.cuda.set_device(local)
    dev = th.device('cuda', local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=dev)
    Bt, Tn, Hn = (8 if args.batch == B_PER_GPU else args.batch), 65536, 40
    lo, hi = shard_of(rank, world, Bt)
    B = hi - lo
    assert B > 0, 'more ranks than sequences'
    d = synthetic.wkv7_inputs(B, Tn, Hn, N, seed=4 + 100 * rank, dtype=th.bfloat16, device=dev, s0_std=0.1)
    ins = [d[n] for n in 'rwkvab']
    step = lambda: attn(*ins, N, s0=d['s0'], return_state=True)
    for _ in range(max(args.warmup, 3)):
        y, sT = step()
    th.cuda.synchronize()
    if dist:
        dist.barrier()
    th.cuda.synchronize()
    e0, e1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(args.steps):
            y, sT = step()
        e1.record()
        th.cuda.synchronize()
    if dist:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist:
        ms = max_over_ranks(ms, dist, dev)
    ms /= args.steps
    # the same call with the chains of the last, partly filled round of SMs cut in time (a no-op split where the shard has no such tail)
    tstep = lambda: attn(*ins, N, s0=d['s0'], return_state=True, time_split='tail')
    with th.no_grad():
        for _ in range(2):
            tstep()
        th.cuda.synchronize()
        if dist:
            dist.barrier()
        e0.record()
        for _ in range(args.steps):
            tstep()
        e1.record()
        th.cuda.synchronize()
    tms = e0.elapsed_time(e1)
    if dist:
        tms = max_over_ranks(tms, dist, dev)
    tms /= args.steps
    finite = bool(th.isfinite(sT).all()) and bool(th.isfinite(y[:, -1]).all())
    status = _lib.device_status()
    if rank == 0:
        peak, which = hbm_peak()
        alg = Bt * Tn * Hn * FWD_BYTES_PER_TOKEN_HEAD
        print(json.dumps({
            'metric': f'WKV7 prefill forward B{Bt} T{Tn} H{Hn} N{N} bf16, s0 -> sT (config 4), Mtokens/s', 'value': Bt * Tn / (ms * 1e-3) / 1e6,
            'unit': 'Mtokens/s', 'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms,
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': f'WKV7 prefill forward B{Bt} T{Tn} H{Hn} N{N} (config 4)', 'global_batch': Bt,
                       'parallelism': f'batch-sharded x{world} ({B} sequences = {B * Hn} chains per GPU), no collective',
                       'l2': 'inputs (6 x 2.7 GB / N) exceed the 126 MB L2; no explicit flush'},
            'roofline': {'bound': 'hbm', 'kernel': 'wkv7_fwd_tc_kernel (tcgen05)', 'achieved': alg / world / (ms * 1e-3) / 1e9, 'peak': peak,
                         'unit': 'GB/s', 'frac': alg / world / (ms * 1e-3) / 1e9 / peak, 'peak_source': which,
                         'algorithmic_bytes': alg // world, 'traffic': None, 'note': 'per GPU'},
            'tail_split': {'ms_per_step': tms, 'value': Bt * Tn / (tms * 1e-3) / 1e6, 'note': "attn(..., time_split='tail')"},
            'gpu_launches': args.steps, 'clocks': clocks.summary(), 'finite': finite, 'device_status': status}))
    if dist:
        dist.destroy_process_group()


def run_reference_cuda(args):
    """The reference's own CUDA kernels (its attn.cu / attn_ln.cu, installed unmodified under baseline/_ref and built
    there for sm_100 through its own load_attn), timed device-resident with CUDA events at the config-1 shape.  Runs
    in this process with baseline/_ref first on sys.path, so nothing of this repository's package is imported.  Not
    the arm the driver's ratio uses (that is `--impl reference`, the CPU path): a second baseline for context."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    ref = os.path.join(ROOT, 'baseline', '_ref')
    op = 'attn_ln' if args.workload == 'attn_ln' else 'attn'
    src = os.path.join(ref, 'wind_rwkv', 'rwkv7', 'attn.cu')
    if not os.path.exists(src) or not th.cuda.is_available():
        print(json.dumps({'impl': 'reference-cuda', 'unavailable': 'baseline/_ref (the reference install with its .cu sources) or a GPU is missing'}))
        return
    sys.path[:] = [p for p in sys.path if not p.endswith('wind-rwkv7_b200')]
    sys.path.insert(0, ref)
    os.environ.setdefault('TORCH_CUDA_ARCH_LIST', '10.0')
    os.environ.setdefault('TORCH_EXTENSIONS_DIR', os.path.join(ref, '_build_' + op))
    Fn = th.nn.functional
    dev = th.device('cuda', 0)
    th.cuda.set_device(0)
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)   # the extension build is verbose on stdout (ninja and nvcc too): keep the JSON line alone there
    try:
        if op == 'attn':
            from wind_rwkv.rwkv7.rwkv7_attn import attn as fn, load_attn
            load_attn(N)
            B, Tn, Hn = args.batch, T, H
        else:
            from wind_rwkv.rwkv7.rwkv7_attn_ln import attn_ln as fn, load_attn_ln
            load_attn_ln(N)
            B, Tn, Hn = (16 if args.batch == B_PER_GPU else args.batch), 4096, 32
    except Exception as e:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps({'impl': 'reference-cuda', 'unavailable': 'building or loading the reference extension failed: ' + repr(e)[:200]}))
        return
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    gen = th.Generator(device=dev).manual_seed(1)
    rn = lambda *sh: th.randn(*sh, generator=gen, device=dev)
    r, k, v = [rn(B, Tn, Hn * N).bfloat16().requires_grad_() for _ in range(3)]
    w = (rn(B, Tn, Hn * N) * 0.5 - 0.6).bfloat16().requires_grad_()
    kap = Fn.normalize(rn(B, Tn, Hn, N), dim=-1).view(B, Tn, Hn * N)
    a = (-kap).bfloat16().requires_grad_()
    b = (kap * th.sigmoid(rn(B, Tn, Hn * N))).bfloat16().requires_grad_()
    ins = [r, w, k, v, a, b]
    if op == 'attn_ln':
        ins += [th.sigmoid(rn(B, Tn, Hn * N)).bfloat16().requires_grad_(), rn(3, Hn * N).requires_grad_()]
    dy = rn(B, Tn, Hn * N).bfloat16()

    def step():
        fn(*ins, N).backward(dy)
        for x in ins:
            x.grad = None
    for _ in range(max(args.warmup, 3)):
        step()
    th.cuda.synchronize()
    steps = max(1, min(args.steps, 50))
    e0, e1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        th.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    print(json.dumps({'impl': 'reference-cuda', 'metric': METRIC if op == 'attn' else 'attn_ln fwd+bwd Mtokens/s', 'value': B * Tn / (ms * 1e-3) / 1e6,
                      'unit': 'Mtokens/s', 'n_gpus': 1, 'steps': steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms,
                      'higher_is_better': True, 'dtype': 'bf16', 'data': 'synthetic',
                      'config': {'workload': f'reference {op} fwd+bwd B{B} T{Tn} H{Hn} N{N} through its own Python entry point '
                                             '(includes its zero-fills and allocations, as a user of it pays them)'},
                      'clocks': clocks.summary()}))


def run_ours(args):
    from wind_rwkv.rwkv7 import _lib, attn, synthetic
    from wind_rwkv.rwkv7.rwkv7_attn import bw_attn, fw_attn

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    assert th.cuda.is_available(), 'bench.py measures the CUDA path; there is no CPU fallback'
    th.cuda.set_device(local)
    dev = th.device('cuda', local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=dev)

    B = args.batch
    d = synthetic.wkv7_inputs(B, T, H, N, seed=1 + rank, dtype=th.bfloat16, device=dev)
    w, r, k, v, a, b = [d[n].view(B, T, H, N) for n in 'wrkvab']
    dy = d['dy'].view(B, T, H, N)
    ev = lambda: th.cuda.Event(enable_timing=True)

    def step(evs=None):
        if evs:
            evs[0].record()
        y, sT, s = fw_attn(w, r, k, v, a, b, None)
        if evs:
            evs[1].record()
        g = bw_attn(w, r, k, v, a, b, s, dy, None, sT)
        if evs:
            evs[2].record()
        return y, g

    for _ in range(max(args.warmup, 3)):
        step()
    th.cuda.synchronize()
    if dist:
        dist.barrier()
    th.cuda.synchronize()
    evs = [[ev(), ev(), ev()] for _ in range(args.steps)]
    t_start, t_end = ev(), ev()
    with ClockSampler(local) as clocks:
        t_start.record()
        for i in range(args.steps):
            step(evs[i])
        t_end.record()
        th.cuda.synchronize()
    if dist:
        dist.barrier()
    th.cuda.synchronize()
    total_ms = t_start.elapsed_time(t_end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    if dist:
        total_ms = max_over_ranks(total_ms, dist, dev)
    ms_per_step = total_ms / args.steps
    value = world * B * T / (ms_per_step * 1e-3) / 1e6

    # end to end through the public API with host buffers: H2D of r,w,k,v,a,b,dy from pinned memory,
    # attn() forward + autograd backward, D2H of y and the six gradients.
    numa = bind_to_gpu_numa_node(local)
    host_in = {n: d[n].cpu().pin_memory() for n in list('rwkvab') + ['dy']}
    host_out = [th.empty(B, T, H * N, dtype=th.bfloat16).pin_memory() for _ in range(7)]

    # Three streams: host->device copies, compute, device->host copies, so that the PCIe transfers of
    # neighbouring steps overlap each other and the kernels.  Every step still moves its own inputs
    # in and its own results out; device input buffers alternate between two sets.
    s_in, s_out, s_cmp = th.cuda.Stream(dev), th.cuda.Stream(dev), th.cuda.current_stream(dev)
    dev_in = [{n: th.empty_like(d[n]) for n in host_in} for _ in range(2)]
    free_ev = [None, None]   # compute of the step that last used buffer set i has finished
    out_ev = [None]

    def e2e_step(i=[0]):
        k = i[0] & 1
        i[0] += 1
        with th.cuda.stream(s_in):
            if free_ev[k] is not None:
                s_in.wait_event(free_ev[k])
            for n in host_in:
                dev_in[k][n].copy_(host_in[n], non_blocking=True)
            ready = th.cuda.Event()
            ready.record(s_in)
        s_cmp.wait_event(ready)
        ins = [dev_in[k][n].detach().requires_grad_() for n in 'rwkvab']
        y = attn(*ins, N)
        y.backward(dev_in[k]['dy'])
        done = th.cuda.Event()
        done.record(s_cmp)
        free_ev[k] = done
        outs = [y.detach()] + [x.grad for x in ins]
        with th.cuda.stream(s_out):
            s_out.wait_event(done)
            for dst, src in zip(host_out, outs):
                src.record_stream(s_out)
                dst.copy_(src, non_blocking=True)
            out_ev[0] = th.cuda.Event()
            out_ev[0].record(s_out)

    def e2e_drain():
        if out_ev[0] is not None:
            s_cmp.wait_event(out_ev[0])

    e2e_steps = 0 if args.no_e2e else max(2, min(args.steps, 10))
    for _ in range(2 if e2e_steps else 0):
        e2e_step()
    e2e_drain()
    th.cuda.synchronize()
    if dist:
        dist.barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()
    e1.record()
    th.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) if e2e_steps else float('inf')
    if dist:
        e2e_ms = max_over_ranks(e2e_ms, dist, dev)
    e2e_value = world * B * T / (e2e_ms / max(e2e_steps, 1) * 1e-3) / 1e6
    nbytes = B * T * H * N * 2
    status = _lib.device_status()

    if rank == 0:
        peak, which = hbm_peak()
        bwd_bytes = B * T * H * BWD_BYTES_PER_TOKEN_HEAD
        fwd_bytes = B * T * H * FWD_BYTES_PER_TOKEN_HEAD
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        line = {
            'metric': METRIC, 'value': value, 'unit': 'Mtokens/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': f'WKV7 fwd+bwd B{B} per GPU T{T} H{H} N{N}, bf16 in/out, fp32 state (config 1)',
                       'global_batch': world * B, 'parallelism': f'batch-sharded x{world}, no collective',
                       'l2': 'inputs (7 x 100 MB) and outputs exceed the 126 MB L2; no explicit flush',
                       'precision': 'single-TF32 tensor-core products, fp32 accumulate'},
            'roofline': {'bound': 'hbm', 'kernel': 'wkv7_bwd_kernel', 'achieved': achieved, 'peak': peak,
                         'unit': 'GB/s', 'frac': achieved / peak, 'peak_source': which,
                         'traffic': BWD_DRAM_TRAFFIC_BYTES, 'algorithmic_bytes': bwd_bytes,
                         'kernel_ms': bwd_ms,
                         'fwd': {'kernel': 'wkv7_fwd_tc_kernel (tcgen05)' if _lib.lib().wkv7_get_fwd_impl() else 'wkv7_fwd_kernel (mma.sync)',
                                 'kernel_ms': fwd_ms, 'algorithmic_bytes': fwd_bytes,
                                 'achieved': fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                 'frac': fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                         'step_frac': (fwd_bytes + bwd_bytes) / (ms_per_step * 1e-3) / 1e9 / peak},
            'e2e': {'value': e2e_value, 'unit': 'Mtokens/s', 'h2d_bytes_per_step': 7 * nbytes,
                    'd2h_bytes_per_step': 7 * nbytes, 'steps': e2e_steps, 'per_gpu': e2e_value / world,
                    'host_buffers': {'pinned': True, 'numa': numa},
                    'note': 'bound by the host link: 1.41 GB cross PCIe per step and GPU, against 2.0 GB of HBM traffic'},
            'gpu_launches': 2 * args.steps,
            'clocks': clocks.summary(),
            'device_status': status,
        }
        if world == 1 and not args.no_secondary:
            # the other workloads of the path, a few steps each (device-resident, whole op forward + backward), so that
            # their numbers are measured by the same run as the headline
            del host_in, host_out, dev_in
            th.cuda.empty_cache()
            sec = {}
            for wl in ('attn_ln', 'prefill', 'prefill_b1', 'ddlerp', 'expand_loras', 'mixer'):
                try:
                    ol = other_line(wl, None, 5, 3)
                    sec[wl] = {'workload': ol['config']['workload'], 'value': ol['value'], 'unit': ol['unit'], 'ms_per_step': ol['ms_per_step'],
                               'roofline_frac': None if ol['roofline'] is None else ol['roofline']['frac'], 'steps': 5}
                    for extra in ('cuda_graph', 'tail_split', 'unsplit_ms_per_step'):
                        if extra in ol:
                            sec[wl][extra] = ol[extra]
                except Exception as e:
                    sec[wl] = {'error': repr(e)[:200]}
                th.cuda.empty_cache()
            line['secondary'] = sec
        if world == 1 and not args.no_cpu_baseline:
            sample_B = 4
            val, sec = cpu_reference_run(sample_B, 2, 1)
            line['cpu_baseline'] = {
                'value': val, 'unit': 'Mtokens/s', 'cores': th.get_num_threads(), 'kind': 'port',
                'sample': f'B={sample_B} of {B}, T={T}, H={H}: torch fp32 per-step recurrence (the reference\'s '
                          f'ref_attn restated), forward + autograd backward, {sec:.1f} s per pass (1 warm-up + 2 timed)'}
        print(json.dumps(line))
    if dist:
        dist.destroy_process_group()


def other_line(wl, batch, steps, warmup):
    """Secondary workloads (not the headline value): device-resident, forward + backward through the
    public API, CUDA events, algorithmic-byte roofline.  Returns the JSON-able line."""
    from wind_rwkv.rwkv7 import TimeMixer, attn, attn_ln, ddlerp, expand_loras, synthetic
    dev = th.device('cuda', th.cuda.current_device())
    gen = th.Generator(device=dev).manual_seed(3)
    rn = lambda *sh, std=1.0: th.randn(*sh, generator=gen, device=dev) * std
    bf = th.bfloat16

    class args:  # the shapes below read args.batch; None selects each workload's own batch
        pass
    args.batch = B_PER_GPU if batch is None else batch
    args.steps, args.warmup = steps, warmup
    if wl == 'attn_ln':      # config 2: B16 T4096 H32
        B, Tn, Hn = args.batch if args.batch != B_PER_GPU else 16, 4096, 32
        d = synthetic.wkv7_inputs(B, Tn, Hn, N, seed=2, dtype=bf, device=dev)
        g, params = synthetic.attn_ln_extras(B, Tn, Hn, N, seed=2, dtype=bf, device=dev)
        ins = [d[n].requires_grad_() for n in 'rwkvab'] + [g.requires_grad_(), params.requires_grad_()]
        fwd = lambda: attn_ln(*ins, N)
        gouts = [d['dy']]
        tokens, alg = B * Tn, B * Tn * Hn * (8 + 15) * N * 2
        name = f'attn_ln fwd+bwd B{B} T{Tn} H{Hn} N{N} bf16 (config 2)'
    elif wl == 'prefill':    # config 4: forward only with state carry
        B, Tn, Hn = args.batch if args.batch != B_PER_GPU else 8, 65536, 40
        d = synthetic.wkv7_inputs(B, Tn, Hn, N, seed=4, dtype=bf, device=dev, s0_std=0.1)
        ins = [d[n] for n in 'rwkvab']
        fwd = lambda: attn(*ins, N, s0=d['s0'], return_state=True)[0]
        gouts = None
        tokens, alg = B * Tn, B * Tn * Hn * 7 * N * 2
        name = f'WKV7 prefill forward B{B} T{Tn} H{Hn} N{N} bf16, s0 -> sT (config 4)'
    elif wl == 'prefill_b1':  # one sequence of a 12-head model: 12 chains for 148 SMs; the sequence runs as 16 parallel segments
        B, Tn, Hn = 1, 65536, 12
        d = synthetic.wkv7_inputs(B, Tn, Hn, N, seed=4, dtype=bf, device=dev, s0_std=0.1)
        ins = [d[n] for n in 'rwkvab']
        fwd = lambda: attn(*ins, N, s0=d['s0'], return_state=True, time_split=16)[0]
        gouts = None
        tokens, alg = B * Tn, B * Tn * Hn * 7 * N * 2
        name = f'WKV7 prefill forward B{B} T{Tn} H{Hn} N{N} bf16, s0 -> sT, time_split=16'
    elif wl == 'ddlerp':
        B, Tn, C, D = args.batch if args.batch != B_PER_GPU else 32, 1024, 768, 32
        x = rn(B, Tn, C).to(bf).requires_grad_()
        prm = [rn(C, std=0.3).requires_grad_(), rn(4 * D, C, std=0.02).requires_grad_(), rn(4, C, D, std=0.02).requires_grad_(),
               rn(4, 1, 1, C, std=0.3).requires_grad_()]
        ins = [x] + prm
        fwd = lambda: ddlerp(*ins)
        gouts = [rn(B, Tn, C).to(bf) for _ in range(4)]
        tokens, alg = B * Tn, B * Tn * 22 * C
        name = f'ddlerp fwd+bwd B{B} T{Tn} C{C} D{D} bf16'
    elif wl == 'expand_loras':
        B, Tn, C, D = args.batch if args.batch != B_PER_GPU else 32, 1024, 768, 16
        acts = [rn(B, Tn, C).to(bf).requires_grad_() for _ in range(2)] + [rn(B, Tn, D).to(bf).requires_grad_() for _ in range(4)]
        prm = [rn(C, D, std=0.1).requires_grad_() for _ in range(4)] + [rn(C, std=0.5).requires_grad_() for _ in range(4)]
        ins = acts + prm
        fwd = lambda: expand_loras(*ins, N)
        gouts = [rn(B, Tn, C).to(bf) for _ in range(4)]
        tokens, alg = B * Tn, B * Tn * (28 * C + 24 * D)
        name = f'expand_loras fwd+bwd B{B} T{Tn} C{C} D{D} bf16'
    elif wl == 'mixer':      # config 3
        from collections import namedtuple
        B, Tn, C = args.batch if args.batch != B_PER_GPU else 32, 1024, 768
        th.manual_seed(0)
        model = TimeMixer(namedtuple('Config', ['n_layer', 'n_head', 'n_embd'])(12, C // N, C), 3).to(dev)
        with th.no_grad():
            for prm_ in model.parameters():
                prm_.add_(th.randn_like(prm_) * 0.02)
        x = rn(B, Tn, C).requires_grad_()
        ins = [x] + list(model.parameters())
        fwd = lambda: model(x)
        gouts = [rn(B, Tn, C).to(bf)]
        tokens, alg = B * Tn, None
        name = f'TimeMixer layer fwd+bwd B{B} T{Tn} d{C} H{C // N} bf16 (config 3)'
    else:
        raise ValueError(wl)

    def step():
        out = fwd()
        if gouts is not None:
            outs = out if isinstance(out, tuple) else (out,)
            th.autograd.backward(outs, gouts)
            for t in ins:
                t.grad = None

    for _ in range(max(args.warmup, 3)):
        step()
    th.cuda.synchronize()
    e0, e1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
    with ClockSampler(th.cuda.current_device()) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        th.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # The small ops are launch-bound in eager mode (a step is a dozen launches of 25-250 us behind Python autograd code):
    # the same step captured once in a CUDA graph and replayed shows what the kernels take without the host in the way.
    graph_ms = None
    if gouts is not None:
        try:
            side = th.cuda.Stream()
            side.wait_stream(th.cuda.current_stream())
            with th.cuda.stream(side):
                step()
            th.cuda.current_stream().wait_stream(side)
            graph = th.cuda.CUDAGraph()
            with th.cuda.graph(graph):
                step()
            for _ in range(3):
                graph.replay()
            th.cuda.synchronize()
            g0, g1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(args.steps):
                graph.replay()
            g1.record()
            th.cuda.synchronize()
            graph_ms = g0.elapsed_time(g1) / args.steps
            del graph
        except Exception as e:  # capture is an extra: report why it was not possible and keep the eager number
            graph_ms = None
            graph_err = repr(e)[:160]
    peak, which = hbm_peak()
    line = {'metric': name + ', Mtokens/s', 'value': tokens / (ms * 1e-3) / 1e6, 'unit': 'Mtokens/s', 'n_gpus': 1,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms, 'higher_is_better': True,
            'dtype': 'bf16', 'data': 'synthetic', 'config': {'workload': name},
            'roofline': None if alg is None else {'bound': 'hbm', 'achieved': alg / (ms * 1e-3) / 1e9, 'peak': peak, 'unit': 'GB/s',
                                                   'frac': alg / (ms * 1e-3) / 1e9 / peak, 'peak_source': which,
                                                   'algorithmic_bytes': alg, 'note': 'whole step (all kernels of the op, forward and backward)'},
            'clocks': clocks.summary()}
    if wl == 'prefill':  # the same call with the chains of the last, partly filled round of SMs cut in time
        with th.no_grad():
            tl = lambda: attn(*ins, N, s0=d['s0'], return_state=True, time_split='tail')
            for _ in range(2):
                tl()
            th.cuda.synchronize()
            u0, u1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
            u0.record()
            for _ in range(3):
                tl()
            u1.record()
            th.cuda.synchronize()
        tms = u0.elapsed_time(u1) / 3
        line['tail_split'] = {'ms_per_step': tms, 'value': tokens / (tms * 1e-3) / 1e6, 'roofline_frac': alg / (tms * 1e-3) / 1e9 / peak,
                              'note': "attn(..., time_split='tail')"}
    if wl == 'prefill_b1':  # the same sequence as one chain per head, for comparison
        with th.no_grad():
            one = lambda: attn(*ins, N, s0=d['s0'], return_state=True)
            one()
            th.cuda.synchronize()
            u0, u1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
            u0.record()
            for _ in range(3):
                one()
            u1.record()
            th.cuda.synchronize()
        line['unsplit_ms_per_step'] = u0.elapsed_time(u1) / 3
    if gouts is not None:
        line['cuda_graph'] = ({'ms_per_step': graph_ms, 'value': tokens / (graph_ms * 1e-3) / 1e6,
                               'roofline_frac': None if alg is None else alg / (graph_ms * 1e-3) / 1e9 / peak}
                              if graph_ms else {'unavailable': graph_err})
    return line


def run_proj(args):
    """The projection GEMM (wkv7_proj_gemm through proj()) at the time mixer's shapes, beside the torch call it replaces
    (a cuBLAS product, plus an elementwise tanh pass where the LoRA's first stage has one).  Forward only, CUDA events,
    one JSON line per shape."""
    from wind_rwkv.rwkv7 import proj
    th.cuda.set_device(0)
    dev = th.device('cuda', 0)
    M = 32 * 1024
    flush = th.empty(256 * 1024 * 1024, dtype=th.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        th.cuda.synchronize()
        e0, e1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        tot = 0.0
        for _ in range(args.steps):
            flush.zero_()   # L2 flush between timed calls
            e0.record()
            fn()
            e1.record()
            th.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / args.steps * 1e3

    with th.no_grad():
        for (N_, K_, tanh) in [(128, 768, (0, 128)), (96, 768, (0, 64)), (768, 768, None), (768, 128, None)]:
            th.manual_seed(0)
            A = th.randn(M, K_, device=dev).bfloat16()
            W = (th.randn(N_, K_, device=dev) / K_ ** 0.5).bfloat16()

            def torch_ref():
                y = A @ W.mT
                if tanh:
                    y[:, tanh[0]:tanh[1]] = th.tanh(y[:, tanh[0]:tanh[1]])
                return y
            ours, ref = timed(lambda: proj(A, W, tanh)), timed(torch_ref)
            err = (proj(A, W, tanh).float() - torch_ref().float()).abs().max().item()
            print(json.dumps({'metric': f'projection GEMM M{M} N{N_} K{K_} bf16' + (f' tanh on columns {tanh}' if tanh else ''), 'unit': 'us',
                              'value': ours, 'torch_cublas_us': ref, 'tflops': 2 * M * N_ * K_ / ours / 1e6, 'max_abs_diff_vs_torch': err,
                              'steps': args.steps, 'higher_is_better': False, 'dtype': 'bf16', 'data': 'synthetic',
                              'config': {'workload': 'proj', 'l2': 'flushed by zeroing a 256 MB buffer before each timed call'}}))


def run_other(args):
    th.cuda.set_device(0)
    print(json.dumps(other_line(args.workload, None if args.batch == B_PER_GPU else args.batch, args.steps, args.warmup)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=400, help='timed steps (default: a timed region of about 0.6 s)')
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference', 'reference-cuda'],
                    help="reference: the reference's CPU recurrence (the driver's reference arm); reference-cuda: the "
                         "reference's own CUDA kernels from baseline/_ref (context only)")
    ap.add_argument('--no-secondary', action='store_true', help='skip the secondary workloads of the headline line')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true', help='skip the host-buffer leg (profiling runs)')
    ap.add_argument('--batch', type=int, default=B_PER_GPU, help='batch per GPU (default: the benchmark shape)')
    ap.add_argument('--workload', default='wkv7', choices=['wkv7', 'attn_ln', 'prefill', 'prefill_b1', 'ddlerp', 'expand_loras', 'mixer', 'proj'],
                    help='wkv7 (default) is the headline line; the others time secondary workloads on one GPU')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    elif args.impl == 'reference-cuda':
        run_reference_cuda(args)
    elif args.workload == 'proj':
        run_proj(args)
    elif args.workload == 'prefill':
        run_prefill(args)
    elif args.workload != 'wkv7':
        run_other(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
