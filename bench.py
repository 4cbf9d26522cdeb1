"""Benchmark of the SLAYER hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--batch B]

One JSON line on stdout (rank 0).  A "step" is one pass of the named kernel over
one batch of seeded synthetic input.  The default workload is CUBA-LIF forward
(spike + voltage from the dendrite input, one fused kernel) at
[64, 8192, 2000], the shape the 70 %-of-HBM-peak target is stated for.  Inputs
are far larger than the 126 MB L2, so nothing is flushed between iterations.

``value``   kernel-resident throughput: inputs already in HBM, CUDA-event timed.
``e2e``     the same metric through the Python API with HOST buffers: the batch
            is streamed host -> device -> host in batch chunks (pinned memory,
            copies and kernels overlapped on three streams), all inside the
            timed region.
``roofline`` algorithmic bytes per launch / mean launch time vs the measured HBM
            copy bandwidth of this pool (MEASURED_PEAKS.json).
``cpu_baseline`` the CPU oracle (a C port of lava-dl's Python loops, OpenMP on
            all host cores) on a bounded sample of the same workload.

With N > 1 every rank runs the full single-GPU workload on its own batch shard
(weak scaling, no forward communication); the fwd+bwd leg all-reduces the
shared decay gradients once per step over NCCL.

``--impl reference`` times the CPU oracle alone (rank 0 only).
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, 'lava-dl_b200')):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

W_SCALE = 4096
THR = 1.25 + 0.01 / 4096

# DRAM bytes per unit (dram__bytes_read.sum + dram__bytes_write.sum over the units
# of the launch) of each workload's kernel, from the batch-8 ncu captures
# summarised under profiles/.  Rows are independent, so traffic grows in
# proportion to the batch: roofline.traffic = this figure x the units of a launch.
NCU_TRAFFIC_PER_UNIT = {
    'cuba_fwd': 11.70,
    'cuba_bwd': 11.88,
    'alif_fwd': 15.28,
    'alif_bwd': 15.84,
    'adrf_fwd': 24.16,
    'adrf_bwd': 24.23,
    'li_fwd': 7.76,
    'li_bwd': 7.74,
    'shift': 7.63,
    'fir_conv': 7.76,
    'delay_fir_fwd': 7.75,
    'sigma_fwd': 7.75,
    'delta_fwd': 7.74,
    'sdnn_fwd': 7.75,
    'cuba_fwd_delayed': 11.70,
}


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------
class Workload:
    """name, default shape, algorithmic bytes per unit and the kernels to run."""

    def __init__(self, name, shape, bytes_per_unit, unit='neuron-steps/s'):
        self.name, self.shape, self.bpu, self.unit = name, shape, bytes_per_unit, unit

    def units(self, shape):
        if self.name.startswith('cfg4'):
            return shape[0] * shape[-1] * CFG4_NEURONS
        return int(np.prod(shape))


def make_inputs(name, shape, device, seed):
    """Seeded synthetic inputs with the value distributions of the benchmark configs."""
    g = torch.Generator(device=device).manual_seed(seed)
    B = shape[0]

    def randn(mean, std):
        return torch.empty(shape, device=device).normal_(mean, std, generator=g)

    d = {}
    if name.startswith('sigma') or name.startswith('sdnn'):
        d['x'] = randn(0.01, 0.1)
    elif name.startswith('delta'):
        d['x'] = randn(0.0, 0.5)
    elif name.startswith('cuba'):
        d['x'] = randn(0.3, 1.0)
    elif name.startswith('alif'):
        d['x'] = randn(0.2, 1.0)
    elif name.startswith('adrf') or name.startswith('rf'):
        d['re'] = randn(0.0, 0.5)
        d['im'] = randn(0.0, 0.5)
    elif name.startswith('delay_fir') or name.startswith('shift') or name.startswith('fir'):
        d['x'] = (torch.rand(shape, device=device, generator=g) < 0.05).float()
        d['delay'] = torch.randint(0, 63, (shape[1],), device=device, generator=g).float()
        d['filter'] = (torch.exp(-torch.arange(64, device=device).float() / 8) / 8)
    if 'bwd' in name:
        d['g'] = randn(0.0, 1.0)
    return d


WORKLOADS = {
    # headline: fused CUBA forward, x in, spike + voltage out = 12 B per neuron-step
    'cuba_fwd': Workload('cuba_fwd', (64, 8192, 2000), 12),
    'cuba_fwd_cfg0': Workload('cuba_fwd_cfg0', (16, 512, 1000), 12),
    # block output path: spikes written one step late plus a per-neuron axonal delay of 0..62 steps, same 12 B
    'cuba_fwd_delayed': Workload('cuba_fwd_delayed', (64, 8192, 2000), 12),
    # backward of the same: g_spike + voltage in, g_x out
    'cuba_bwd': Workload('cuba_bwd', (64, 8192, 2000), 12),
    'alif_fwd': Workload('alif_fwd', (64, 4096, 2000), 16),
    'alif_bwd': Workload('alif_bwd', (64, 4096, 2000), 16),
    'adrf_fwd': Workload('adrf_fwd', (64, 8192, 1000), 24),
    'adrf_bwd': Workload('adrf_bwd', (64, 8192, 1000), 24),
    'li_fwd': Workload('li_fwd', (64, 8192, 2000), 8),
    'li_bwd': Workload('li_bwd', (64, 8192, 2000), 8),
    # sigma-delta family (next to the path): running sum, delta encoder, fused relu neuron, 8 B per step each
    'sigma_fwd': Workload('sigma_fwd', (64, 8192, 2000), 8),
    'delta_fwd': Workload('delta_fwd', (64, 8192, 2000), 8),
    'delta_bwd': Workload('delta_bwd', (64, 8192, 2000), 8),
    'sdnn_fwd': Workload('sdnn_fwd', (64, 8192, 2000), 8),
    'shift': Workload('shift', (128, 16384, 1000), 8, 'elements/s'),
    'fir_conv': Workload('fir_conv', (128, 16384, 1000), 8, 'elements/s'),
    'delay_fir_fwd': Workload('delay_fir_fwd', (128, 16384, 1000), 8, 'elements/s'),
    'delay_fir_bwd': Workload('delay_fir_bwd', (128, 16384, 1000), 8, 'elements/s'),
}
# full CUBA conv network of the last benchmark config (blocks = this library's synapse kernels + fused neuron kernel +
# one-step delay); units = neuron-steps over all seven spiking layers (33291 neurons per sample)
WORKLOADS['cfg4_fwd'] = Workload('cfg4_fwd', (32, 2, 128, 128, 300), 0)
WORKLOADS['cfg4_train'] = Workload('cfg4_train', (32, 2, 128, 128, 300), 0)
# dense recurrent CUBA block (block.cuba.Recurrent, 512 -> 512 neurons): one launch per direction for the walk over time
WORKLOADS['recurrent_fwd'] = Workload('recurrent_fwd', (128, 512, 300), 0)
WORKLOADS['recurrent_train'] = Workload('recurrent_train', (128, 512, 300), 0)
# the same block walked the way the reference does it (utils/recurrent.py:17-32): one matmul and one
# neuron call with a single time step per step, here on this library's own neuron kernel
WORKLOADS['recurrent_fwd_stepwise'] = Workload('recurrent_fwd_stepwise', (128, 512, 300), 0)
NETWORKS = ('cfg4', 'recurrent')   # chains of kernels: no single roofline, no CPU port
CFG4_NEURONS = 2048 + 16384 + 4096 + 8192 + 2048 + 512 + 11


def build_step(name, shape, device, seed):
    """Returns (step_fn, launches_per_step, keepalive).  step_fn launches the kernel(s)
    of one step on the current stream and returns nothing."""
    from lava_dl_b200 import _ops
    d = make_inputs(name, shape, device, seed)
    C = shape[1]
    lead = shape[:-1]
    one = lambda v: torch.tensor([float(v)], device=device)  # noqa: E731
    zeros = torch.zeros(lead, device=device)

    if name.startswith('cfg4'):
        import lava_dl_b200.slayer as slayer
        from lava_dl_b200 import _dist
        train = name == 'cfg4_train'
        p = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03)
        blk = slayer.block.cuba
        torch.manual_seed(seed)
        net = torch.nn.ModuleList([
            blk.Pool(p, 4), blk.Conv(p, 2, 16, 5, padding=2), blk.Pool(p, 2), blk.Conv(p, 16, 32, 3, padding=1),
            blk.Pool(p, 2), blk.Flatten(), blk.Dense(p, 2048, 512), blk.Dense(p, 512, 11),
        ]).to(device)
        for layer in net:
            if hasattr(layer, 'synapse') and layer.synapse.weight.requires_grad:
                torch.nn.init.normal_(layer.synapse.weight, 0.0, 0.1)
        gen = torch.Generator(device=device).manual_seed(seed)
        x = (torch.rand(shape, device=device, generator=gen) < 0.02).float()
        params = [q for q in net.parameters() if q.requires_grad]

        def forward():
            y = x
            for layer in net:
                y = layer(y)
            return y

        if not train:
            def step():
                with torch.no_grad():
                    return forward()
            return step, 10, (net, x)  # 7 fused neuron kernels (delay folded in) + 3 pooling kernels

        def step():
            for q in params:
                q.grad = None
            forward().sum().backward()
            _dist.allreduce_param_grads(params)
        # forward as above, backward: 7 fused neuron kernels + 3 pooling adjoints
        return step, 20, (net, x)
    if name.startswith('recurrent'):
        import lava_dl_b200.slayer as slayer
        from lava_dl_b200 import _dist
        train = name == 'recurrent_train'
        torch.manual_seed(seed)
        blk = slayer.block.cuba.Recurrent(dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03),
                                          shape[1], shape[1], weight_scale=2).to(device)
        gen = torch.Generator(device=device).manual_seed(seed)
        x = (torch.rand(shape, device=device, generator=gen) < 0.05).float()
        params = [q for q in blk.parameters() if q.requires_grad]

        def stepwise():
            with torch.no_grad():
                z = blk.input_synapse(x)
                rec_t = blk.neuron.quantize_8bit(blk.recurrent_synapse.weight.reshape(shape[1], shape[1])).t()
                out = torch.zeros_like(z)
                spike = torch.zeros(z.shape[:-1] + (1,), device=device)
                for t in range(z.shape[-1]):
                    feedback = torch.matmul(spike[..., 0], rec_t)
                    spike = blk.neuron((z[..., t] + feedback).unsqueeze(-1))
                    out[..., t:t + 1] = spike
                return out
        if name == 'recurrent_fwd_stepwise':
            return stepwise, shape[-1], (blk, x)

        def step():
            if not train:
                with torch.no_grad():
                    return blk(x)
            for q in params:
                q.grad = None
            blk(x).sum().backward()
            _dist.allreduce_param_grads(params)
        return step, (2 if train else 1), (blk, x)
    if name == 'sigma_fwd':
        def step():
            return _ops.sigma_fwd(d['x'])
        return step, 1, d
    if name == 'delta_fwd':
        thr = one(0.3)

        def step():
            return _ops.delta_fwd(d['x'], thr, None, None, 4096, want_delta=False)
        return step, 1, d
    if name == 'delta_bwd':
        thr = one(0.3)
        del d['x']

        def step():
            return _ops.delta_bwd(d['g'], None, thr, 1.0, 1.0, False)
        return step, 1, d
    if name == 'sdnn_fwd':
        thr = one(0.1)

        def step():
            return _ops.sdnn_relu_fwd(d['x'], thr, None, None, None, None, 4096)
        return step, 1, d
    if name == 'cuba_fwd_delayed':
        cd, vd = one(1024), one(123)
        gen = torch.Generator(device=device).manual_seed(seed + 1)
        d['delay'] = torch.randint(0, 63, (C,), device=device, generator=gen).float()

        def step():
            return _ops.cuba_fwd(d['x'], cd, vd, zeros, zeros, THR, W_SCALE, want_current=False, want_spike=True,
                                 spike_delay=1, axon_delay=d['delay'])
        return step, 1, d
    if name.startswith('cuba_fwd'):
        cd, vd = one(1024), one(123)

        def step():
            return _ops.cuba_fwd(d['x'], cd, vd, zeros, zeros, THR, W_SCALE, want_current=False, want_spike=True)
        return step, 1, d
    if name == 'cuba_bwd':
        cd, vd = one(1024), one(123)
        r = _ops.cuba_fwd(d['x'], cd, vd, zeros, zeros, THR, W_SCALE, want_current=False, want_spike=True)
        d['voltage'] = r['voltage']
        del d['x'], r

        def step():
            return _ops.cuba_bwd(d['g'], d['voltage'], THR, None, cd, vd, 125.0, 0.1, False, False)
        return step, 1, d
    if name in ('alif_fwd', 'alif_bwd'):
        cd, vd, td, rd = one(819), one(205), one(410), one(410)
        ths = torch.ones(lead, device=device)
        args = (d['x'], cd, vd, rd, td, zeros, zeros, zeros, ths, 0.5, 1.0, W_SCALE)
        if name == 'alif_fwd':
            def step():
                return _ops.alif_fwd(*args, dynamics_mode=False)
            return step, 1, d
        (spk, vol, thsum), _ = _ops.alif_fwd(*args, dynamics_mode=False)
        d.update(voltage=vol, thsum=thsum)
        del d['x'], spk

        def step():
            return _ops.cuba_bwd(d['g'], d['voltage'], d['thsum'], None, cd, vd, 100.0, 0.1, False, False)
        return step, 1, d
    if name in ('adrf_fwd', 'adrf_bwd'):
        gen = torch.Generator(device=device).manual_seed(seed + 1)
        period = 10 + 30 * torch.rand(C, device=device, generator=gen)
        sd = (4096 * torch.sin(2 * np.pi / period) * 0.9).round()
        cdec = (4096 * torch.cos(2 * np.pi / period) * 0.9).round()
        ad = dict(ref_decay=one(410), th_decay=one(410), ref_state=zeros, th_state=0.5 * torch.ones(lead, device=device),
                  th_step=0.25, th0=0.5)
        if name == 'adrf_fwd':
            def step():
                return _ops.rf_fwd(d['re'], d['im'], sd, cdec, zeros, zeros, 0.5, W_SCALE, adaptive=ad)
            return step, 1, d
        outs, _ = _ops.rf_fwd(d['re'], d['im'], sd, cdec, zeros, zeros, 0.5, W_SCALE, adaptive=ad)
        d.update(real=outs[1], imag=outs[2], thsum=outs[3])
        del d['re'], d['im'], outs

        def step():
            return _ops.rf_bwd(d['g'], d['real'], d['imag'], d['thsum'], sd, cdec, 50.0, 0.1, False, False)
        return step, 1, d
    if name == 'li_fwd':
        d['x'] = torch.empty(shape, device=device).normal_(0.3, 1.0)
        dec = one(1024)

        def step():
            return _ops.li_fwd(d['x'], dec, zeros, W_SCALE)
        return step, 1, d
    if name == 'li_bwd':
        dec = one(1024)

        def step():
            return _ops.li_bwd(d['g'], None, dec, False)
        return step, 1, d
    if name == 'shift':
        def step():
            return _ops.shift(d['x'], d['delay'])
        return step, 1, d
    if name == 'fir_conv':
        def step():
            return _ops.fir(d['x'], d['filter'], 1.0, False)
        return step, 1, d
    if name == 'delay_fir_fwd':
        def step():
            return _ops.shift_fir(d['x'], d['delay'], 1, d['filter'], 1.0, backward=False)
        return step, 1, d
    if name == 'delay_fir_bwd':
        def step():
            return _ops.shift_fir(d['g'], d['delay'], 1, d['filter'], 1.0, backward=True)
        return step, 1, d
    raise SystemExit(f'unknown workload {name}')


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Polls NVML (read-only) every few milliseconds between start() and stop():
    SM clock, max SM clock and the active clock-event reasons."""
    REASONS = {0x8: 'hw_slowdown', 0x40: 'hw_thermal_slowdown', 0x20: 'sw_thermal_slowdown', 0x4: 'sw_power_cap'}

    def __init__(self, index):
        self.index, self.sm, self.bits, self.max_sm = index, [], 0, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    @staticmethod
    def _physical_index(index):
        vis = os.environ.get('CUDA_VISIBLE_DEVICES')
        if vis:
            ids = [v.strip() for v in vis.split(',') if v.strip()]
            if index < len(ids) and ids[index].isdigit():
                return int(ids[index])
        return index

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.sm:
            return {'sm_mhz': None, 'sm_max_mhz': self.max_sm, 'reasons': [], 'samples': 0}
        reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        return {'sm_mhz': statistics.median(self.sm), 'sm_max_mhz': self.max_sm, 'reasons': reasons,
                'samples': len(self.sm)}


# ---------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline and --impl reference)
# ---------------------------------------------------------------------------
def cpu_sample_shape(wl):
    """Bounded sample of the workload: same neurons and T, a slice of the batch."""
    b, c, t = wl.shape
    target = 2.0e8  # neuron-steps per timed pass
    bs = max(1, min(b, int(target // (c * t))))
    return (bs, c, t)


def cpu_step_fn(name, shape, seed):
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    if name.startswith('cuba') or name.startswith('li'):
        x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
        g = np.ones(shape, np.float32)
        if name == 'li_fwd':
            return lambda: O.li_fwd(x, np.array([1024.0]), 0.0, W_SCALE)
        if name == 'li_bwd':
            return lambda: O.li_bwd(g, x, np.array([1024.0]))
        if 'bwd' in name:
            vol = O.cuba(x, 1.25, 1024.0, 123.0)['voltage']

            def bwd():
                gv = O.spike_bwd(vol, THR, g, 125.0, 0.1)
                gc, _ = O.li_bwd(gv, vol, np.array([123.0]))
                return O.li_bwd(gc, vol, np.array([1024.0]))
            return bwd
        return lambda: O.cuba(x, 1.25, 1024.0, 123.0)
    if name.startswith('alif'):
        x = rng.normal(0.2, 1.0, size=shape).astype(np.float32)
        g = np.ones(shape, np.float32) if 'bwd' in name else None
        return lambda: O.alif(x, 1.0, 0.5, 819.0, 205.0, 410.0, 410.0, grad_spike=g)
    if name.startswith('adrf'):
        re = rng.normal(0, 0.5, size=shape).astype(np.float32)
        im = rng.normal(0, 0.5, size=shape).astype(np.float32)
        p = rng.uniform(10, 40, size=shape[1])
        sd = np.round(4096 * np.sin(2 * np.pi / p) * 0.9)
        cd = np.round(4096 * np.cos(2 * np.pi / p) * 0.9)
        g = np.ones(shape, np.float32) if 'bwd' in name else None
        return lambda: O.adrf(re, im, 0.5, 0.25, sd, cd, 410.0, 410.0, grad_spike=g)
    x = (rng.uniform(size=shape) < 0.05).astype(np.float32)
    delay = rng.integers(0, 63, size=shape[1]).astype(np.float32)
    f = (np.exp(-np.arange(64) / 8) / 8).astype(np.float32)
    if name == 'shift':
        return lambda: O.shift(x, delay)
    if name == 'fir_conv':
        return lambda: O.conv(x, f)
    if name == 'delay_fir_bwd':
        return lambda: O.shift(O.corr(x, f), -delay)
    return lambda: O.conv(O.shift(x, delay), f)


def time_cpu(wl, steps, warmup, seed=0):
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    shape = cpu_sample_shape(wl)
    fn = cpu_step_fn(wl.name, shape, seed)
    for _ in range(max(1, warmup)):
        fn()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    units = wl.units(shape)
    return {'value': units / sec, 'unit': wl.unit, 'cores': cores, 'kind': 'port',
            'sample': f'{wl.name} on {list(shape)} (batch slice of {list(wl.shape)}), median of {steps} passes, '
                      f'{sec * 1e3:.1f} ms per pass, OpenMP on {cores} threads'}, sec


# ---------------------------------------------------------------------------
# end-to-end (host buffers) through the public API
# ---------------------------------------------------------------------------
def e2e_cuba(shape, device, steps, warmup):
    """Host-resident input -> spikes back on the host, streamed in batch chunks.
    Three streams: H2D, compute, D2H; chunk k+1 uploads while chunk k computes."""
    import lava_dl_b200.slayer as slayer
    B, C, T = shape
    chunk = max(1, min(B, 8))
    nchunks = (B + chunk - 1) // chunk
    try:
        x_host = torch.empty(shape, pin_memory=True)
        s_host = torch.empty(shape, pin_memory=True)
    except RuntimeError:
        return None
    gen = torch.Generator().manual_seed(0)
    for b in range(0, B, chunk):  # fill chunk-wise to bound temporary memory
        x_host[b:b + chunk].normal_(0.3, 1.0, generator=gen)
    neuron = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03).to(device)
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    comp = torch.cuda.current_stream(device)
    xbuf = [torch.empty((chunk, C, T), device=device) for _ in range(2)]
    free_x = [torch.cuda.Event() for _ in range(2)]
    up_done = [torch.cuda.Event() for _ in range(2)]

    def one_pass():
        outs = []
        for k in range(nchunks):
            b0, b1 = k * chunk, min(B, (k + 1) * chunk)
            i = k & 1
            with torch.cuda.stream(up):
                up.wait_event(free_x[i])
                xbuf[i][:b1 - b0].copy_(x_host[b0:b1], non_blocking=True)
                up_done[i].record(up)
            comp.wait_event(up_done[i])
            with torch.no_grad():
                spike = neuron(xbuf[i][:b1 - b0])
            free_x[i].record(comp)
            done = torch.cuda.Event()
            done.record(comp)
            with torch.cuda.stream(down):
                down.wait_event(done)
                s_host[b0:b1].copy_(spike, non_blocking=True)
                spike.record_stream(down)
            outs.append(spike)
        comp.wait_stream(down)
        return outs

    for e in free_x:
        e.record(comp)
    for _ in range(max(1, warmup)):
        one_pass()
    torch.cuda.synchronize(device)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record(comp)
    for _ in range(steps):
        one_pass()
    t1.record(comp)
    torch.cuda.synchronize(device)
    ms = t0.elapsed_time(t1) / steps
    nbytes = int(np.prod(shape)) * 4
    return {'ms': ms, 'h2d': nbytes, 'd2h': nbytes, 'launches': nchunks, 'rate': float(s_host.mean())}


def fwd_bwd_cuba(shape, device, steps, warmup, world):
    """Training step through the public API: spikes, sum-of-spikes loss, backward
    with learnable decays, and (N > 1) one NCCL all-reduce of the decay gradients."""
    import lava_dl_b200.slayer as slayer
    from lava_dl_b200 import _dist
    gen = torch.Generator(device=device).manual_seed(4321)
    x = torch.empty(shape, device=device).normal_(0.3, 1.0, generator=gen).requires_grad_(True)
    neuron = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03,
                                       requires_grad=True).to(device)
    params = list(neuron.parameters())

    def one_step():
        x.grad = None
        for p in params:
            p.grad = None
        neuron(x).sum().backward()
        return _dist.allreduce_param_grads(params)

    for _ in range(max(1, warmup)):
        n_reduced = one_step()
    torch.cuda.synchronize(device)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        one_step()
    t1.record()
    torch.cuda.synchronize(device)
    return t0.elapsed_time(t1) / steps, n_reduced


# ---------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='cuba_fwd', choices=sorted(WORKLOADS))
    ap.add_argument('--batch', type=int, default=0, help='override the batch size (small ncu captures)')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-cpu', action='store_true')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup

    wl = WORKLOADS[args.workload]
    shape = tuple(wl.shape)
    if args.batch > 0:
        shape = (args.batch,) + shape[1:]
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))

    if args.impl == 'reference':
        if rank != 0:
            return
        if wl.name.startswith(NETWORKS):
            print(json.dumps({'impl': 'reference', 'unavailable': 'no CPU port of this workload (a network of kernels)'}))
            return
        cpu, sec = time_cpu(wl, max(1, args.steps), max(1, args.warmup))
        line = {
            'impl': 'reference', 'metric': f'neuron-steps/sec ({wl.name})' if wl.unit.startswith('neuron') else
            f'elements/sec ({wl.name})', 'value': cpu['value'], 'unit': wl.unit, 'n_gpus': args.gpus,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': sec * 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'int32+f32', 'data': 'synthetic',
            'config': {'workload': f'{wl.name} {list(wl.shape)}', 'sample': cpu['sample']},
            'cpu_baseline': cpu,
            'e2e': {'value': cpu['value'], 'unit': wl.unit, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        }
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), 'bench.py needs a CUDA device (no CPU fallback exists)'
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=device)

    step, launches_per_step, keep = build_step(wl.name, shape, device, seed=1234 + rank)
    units = wl.units(shape)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        step()
    barrier()
    stream = torch.cuda.current_stream(device)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local) as clocks:
        barrier()
        evs[0].record(stream)
        for i in range(args.steps):
            step()
            evs[i + 1].record(stream)
        barrier()
    total_ms = evs[0].elapsed_time(evs[-1])
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    if dist is not None:
        t = torch.tensor([total_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = units * world / (ms_per_step * 1e-3)

    peak, peak_kind = peaks()
    kern_ms = statistics.mean(per) / (1 if wl.name.startswith(NETWORKS) else launches_per_step)
    achieved = wl.bpu * units / (kern_ms * 1e-3) / 1e9
    tpu = NCU_TRAFFIC_PER_UNIT.get(wl.name)
    roofline = {'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
                'traffic': None if tpu is None else tpu * units, 'peak_kind': f'of {peak_kind}',
                'algorithmic_bytes_per_unit': wl.bpu, 'kernel_ms': kern_ms, 'kernel_ms_min': min(per),
                'frac_of_nominal_8TBps': achieved / 8000.0}
    if 'fir' in wl.name:
        # 64 taps per 8-byte unit run on the tensor cores (banded matrix product, tcgen05 kind::tf32, three
        # TF32 products per term, two when the input is exact in TF32): the bound is HBM again.  The FP32
        # sliding-window kernel that small or unaligned problems still take is capped by the FMA pipe at
        # SMs x 128 lanes x clock / 64 units per second.
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        clk = (clocks.summary()['sm_mhz'] or 1965.0) * 1e6
        roofline['math'] = 'tcgen05.mma kind::tf32, hi*hi + hi*lo + lo*hi, fp32 accumulate in TMEM'
        roofline['fp32_fma_ceiling_of_simt_kernel_GBps'] = sms * 128 * clk / 64.0 * wl.bpu / 1e9

    line = {
        'metric': f'neuron-steps/sec ({wl.name})' if wl.unit.startswith('neuron') else f'elements/sec ({wl.name})',
        'value': value, 'unit': wl.unit, 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'f32 (3xTF32 products, fp32 accumulate)' if 'fir' in wl.name else 'int32+f32', 'data': 'synthetic',
        'config': {'workload': f'{wl.name} {list(shape)} per GPU', 'global_batch': shape[0] * world,
                   'l2': 'inputs larger than L2 (no flush)', 'parallelism': f'batch shards x{world}, no forward collective'},
        'gpu_launches': args.steps * launches_per_step,
        'roofline': roofline,
        'clocks': clocks.summary(),
    }

    del keep, step
    torch.cuda.empty_cache()

    if wl.name == 'cuba_fwd' and not args.no_e2e:
        r = e2e_cuba(shape, device, steps=max(2, min(args.steps, 5)), warmup=1)
        if r is not None:
            ms = r['ms']
            if dist is not None:
                t = torch.tensor([ms], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            line['e2e'] = {'value': units * world / (ms * 1e-3), 'unit': wl.unit, 'h2d_bytes_per_step': r['h2d'],
                           'd2h_bytes_per_step': r['d2h'], 'ms_per_step': ms,
                           'path': 'slayer.neuron.cuba.Neuron.forward on pinned host batches, chunked over batch',
                           'spike_rate': r['rate']}
    if wl.name == 'cuba_fwd' and not args.no_e2e:
        ms, n_red = fwd_bwd_cuba(shape, device, steps=max(2, min(args.steps, 5)), warmup=2, world=world)
        if dist is not None:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        # bytes: fwd x in, spike + voltage + current out (16); ones-like grad written + read (8);
        # bwd g_spike, voltage, current in, g_x out (16)
        line['fwd_bwd'] = {'value': units * world / (ms * 1e-3), 'unit': wl.unit, 'ms_per_step': ms,
                           'allreduce_elements': n_red,
                           'path': 'cuba.Neuron(requires_grad=True)(x).sum().backward() + one all-reduce of decay grads'}
        torch.cuda.empty_cache()
    if wl.name.startswith('recurrent'):
        line['roofline'] = None  # latency-bound walk over time plus two GEMMs
        line['config']['network'] = 'block.cuba.Recurrent(512, 512), spikes in at 5 %'
    if wl.name.startswith('cfg4'):
        line['roofline'] = None  # a chain of synapse and neuron kernels has no single roof
        line['config']['network'] = 'Pool4-Conv(2,16,5)-Pool2-Conv(16,32,3)-Pool2-Flatten-Dense(2048,512)-Dense(512,11), CUBA'
    if rank == 0 and not args.no_cpu and not wl.name.startswith(NETWORKS):
        cpu, _ = time_cpu(wl, steps=3, warmup=1)
        line['cpu_baseline'] = cpu
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == '__main__':
    main()
