"""Benchmark of the SLAYER hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--batch B]

One JSON line on stdout (rank 0).  A "step" is one pass of the named kernel over
one batch of seeded synthetic input.  The default workload is CUBA-LIF forward
(spike + voltage from the dendrite input, one fused kernel) at
[64, 8192, 2000], the shape the 70 %-of-HBM-peak target is stated for.  Inputs
are far larger than the 126 MB L2, so nothing is flushed between iterations.

``value``   kernel-resident throughput: inputs already in HBM, CUDA-event timed.
``parity``  outside the timed region, the last timed output of the first sample(s) is
            replayed through the CPU oracle on the same input bits: spikes and voltage
            must be identical (``fwd_bwd.parity``: the input gradient of the last step).
``e2e``     the same metric through the Python API with HOST buffers: the batch
            is streamed host -> device -> host in batch chunks (pinned memory on the
            GPU's NUMA node, copies and kernels overlapped on three streams), all
            inside the timed region; ``e2e.host_copy_peak_GBps`` is what plain pinned
            copies of one chunk reach on this host with every rank copying at once,
            ``e2e.packed`` the same pass with the opt-in bit-packed result.
``roofline`` algorithmic bytes per launch / mean launch time vs the measured HBM
            copy bandwidth of this pool (MEASURED_PEAKS.json).
``extra``   (default workload only) the kernels of the other benchmark configurations
            at their full shapes -- ms, GB/s, fraction of the same peak -- and the conv
            network of the last configuration, forward and training step.
``cpu_baseline`` the CPU oracle (a C port of lava-dl's Python loops, OpenMP on
            all host cores) on a bounded sample of the same workload.

With N > 1 every rank runs the full single-GPU workload on its own batch shard
(weak scaling, no forward communication); the fwd+bwd leg all-reduces the
shared decay gradients once per step over NCCL.  The conv network is the
exception: its global batch of 32 is split over the ranks (strong scaling) and
the weight and decay gradients are summed in one flattened all-reduce.

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
    'cuba_fwd_infer': 7.76,
    'cuba_fwd_delayed': 11.70,
    'cuba_bwd': 11.88,
    'alif_fwd': 11.31,
    'alif_fwd_infer': 7.46,
    'alif_bwd': 11.63,
    'adrf_fwd': 19.69,
    'adrf_fwd_infer': 12.01,
    'adrf_bwd': 19.82,
    'li_fwd': 7.75,
    'li_bwd': 7.73,
    'sigma_fwd': 7.74,
    'delta_fwd': 7.74,
    'delta_bwd': 7.74,
    'sdnn_fwd': 7.76,
    'shift': 7.64,
    'fir_conv': 7.76,
    'delay_fir_fwd': 7.75,
    'delay_fir_bwd': 7.76,
    'cuba_fwd_train': 15.67,
    'cuba_bwd_dgrad': 15.99,
    'li_bwd_dgrad': 11.88,
    'ath_fwd': 11.29,
    'apth_fwd': 15.45,
    'res_fwd': 15.70,
    'res_bwd': 15.64,
    'res_bwd_pgrad': 24.21,
    'adres_fwd': 23.63,
    'spike_fwd': 7.67,
    'spike_bwd': 11.76,
    'cspike_fwd': 11.51,
    'cspike_bwd': 19.45,
    'sdnn_bwd': 11.92,
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

    def bytes(self, shape):
        """Algorithmic bytes of one launch."""
        n = int(np.prod(shape))
        if self.name.startswith('pool_'):
            return 4 * (n + n // 16)                       # 4 x 4 windows
        if self.name in ('conv5_fwd',):
            return 4 * (n + n // shape[1] * 16)            # 2 -> 16 channels
        if self.name == 'conv3_fwd':
            return 4 * (n + n // shape[1] * 32)            # 16 -> 32 channels
        if self.name == 'conv3_dgrad':
            return 4 * (n + n // shape[1] * 16)            # gradient of 32 channels -> 16 channels
        if self.name == 'conv3_wgrad':
            return 4 * (n + n // shape[1] * 32)            # input and output gradient read once
        return self.bpu * n


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
    'cuba_fwd_infer': Workload('cuba_fwd_infer', (64, 8192, 2000), 8),   # x in, fp32 spikes out: forward under no_grad
    'cuba_fwd_cfg0': Workload('cuba_fwd_cfg0', (16, 512, 1000), 12),
    # the same through slayer.neuron.cuba.Neuron.forward: the kernel plus the Python / ATen glue of one call
    'cuba_fwd_cfg0_api': Workload('cuba_fwd_cfg0_api', (16, 512, 1000), 12),
    'cuba_fwd_cfg0_graph': Workload('cuba_fwd_cfg0_graph', (16, 512, 1000), 12),   # the same call replayed as a CUDA graph
    # block output path: spikes written one step late plus a per-neuron axonal delay of 0..62 steps, same 12 B
    'cuba_fwd_delayed': Workload('cuba_fwd_delayed', (64, 8192, 2000), 12),
    # backward of the same: g_spike + voltage in, g_x out
    'cuba_bwd': Workload('cuba_bwd', (64, 8192, 2000), 12),
    'alif_fwd': Workload('alif_fwd', (64, 4096, 2000), 12),   # x in; spike and voltage - threshold out (training forward)
    'alif_fwd_infer': Workload('alif_fwd_infer', (64, 4096, 2000), 8),   # x in, fp32 spikes out: forward under no_grad
    'alif_bwd': Workload('alif_bwd', (64, 4096, 2000), 12),   # grad_spike and voltage - threshold in; grad_x out
    'adrf_fwd': Workload('adrf_fwd', (64, 8192, 1000), 20),   # re, im in; spike, re - threshold, im out (training forward)
    'adrf_fwd_infer': Workload('adrf_fwd_infer', (64, 8192, 1000), 12),   # re, im in, fp32 spikes out
    'adrf_bwd': Workload('adrf_bwd', (64, 8192, 1000), 20),   # grad_spike, re - threshold, im in; grad_re, grad_im out
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
# the kernels behind the public dynamics() / spike() calls and the training variants of the fused ones
# (bytes per unit: every tensor the call reads or returns, once)
WORKLOADS.update({
    'cuba_fwd_train': Workload('cuba_fwd_train', (64, 8192, 2000), 16),   # x in; current, voltage, spike out
    'cuba_bwd_dgrad': Workload('cuba_bwd_dgrad', (64, 8192, 2000), 16),   # g_spike, voltage, current in; g_x out
    'li_bwd_dgrad': Workload('li_bwd_dgrad', (64, 8192, 2000), 12),       # g, saved output in; g_x out
    'ath_fwd': Workload('ath_fwd', (64, 4096, 2000), 12),
    'apth_fwd': Workload('apth_fwd', (64, 4096, 2000), 16),
    'res_fwd': Workload('res_fwd', (64, 8192, 1000), 16),
    'res_bwd': Workload('res_bwd', (64, 8192, 1000), 16),
    'res_bwd_pgrad': Workload('res_bwd_pgrad', (64, 8192, 1000), 24),
    'adres_fwd': Workload('adres_fwd', (64, 8192, 1000), 24),
    'spike_fwd': Workload('spike_fwd', (64, 8192, 2000), 8),
    'spike_bwd': Workload('spike_bwd', (64, 8192, 2000), 12),
    'cspike_fwd': Workload('cspike_fwd', (64, 8192, 1000), 12),
    'cspike_bwd': Workload('cspike_bwd', (64, 8192, 1000), 20),
    'sdnn_bwd': Workload('sdnn_bwd', (64, 8192, 2000), 12),               # g, activation in; g_x out
})
# synapse kernels of the conv network at its own layer shapes (units = output elements; bytes per unit
# = output written + input read, scaled to one output element)
WORKLOADS.update({
    'pool_fwd': Workload('pool_fwd', (32, 2, 128, 128, 300), 0, 'elements/s'),
    'pool_bwd': Workload('pool_bwd', (32, 2, 128, 128, 300), 0, 'elements/s'),
    'conv5_fwd': Workload('conv5_fwd', (32, 2, 32, 32, 300), 0, 'elements/s'),     # 2 -> 16, 5 x 5: fp32 kernel
    'conv3_fwd': Workload('conv3_fwd', (32, 16, 16, 16, 300), 0, 'elements/s'),    # 16 -> 32, 3 x 3: tensor cores
    'conv3_dgrad': Workload('conv3_dgrad', (32, 32, 16, 16, 300), 0, 'elements/s'),
    'conv3_wgrad': Workload('conv3_wgrad', (32, 16, 16, 16, 300), 0, 'elements/s'),
})
SYNAPSE = ('pool_', 'conv5_', 'conv3_')
# full CUBA conv network of the last benchmark config (blocks = this library's synapse kernels + fused neuron kernel +
# one-step delay); units = neuron-steps over all seven spiking layers (33291 neurons per sample)
WORKLOADS['cfg4_fwd'] = Workload('cfg4_fwd', (32, 2, 128, 128, 300), 0)
WORKLOADS['cfg4_train'] = Workload('cfg4_train', (32, 2, 128, 128, 300), 0)
WORKLOADS['cfg4_fwd_graph'] = Workload('cfg4_fwd_graph', (32, 2, 128, 128, 300), 0)   # cfg4_fwd replayed as one CUDA graph
# dense recurrent CUBA block (block.cuba.Recurrent, 512 -> 512 neurons): one launch per direction for the walk over time
WORKLOADS['recurrent_fwd'] = Workload('recurrent_fwd', (128, 512, 300), 0)
WORKLOADS['recurrent_train'] = Workload('recurrent_train', (128, 512, 300), 0)
# the same block walked the way the reference does it (utils/recurrent.py:17-32): one matmul and one
# neuron call with a single time step per step, here on this library's own neuron kernel
WORKLOADS['recurrent_fwd_stepwise'] = Workload('recurrent_fwd_stepwise', (128, 512, 300), 0)
NETWORKS = ('cfg4', 'recurrent')   # chains of kernels: no single roofline, no CPU port
# workloads the CPU oracle is timed on (cpu_baseline, --impl reference)
CPU_PORTED = ('cuba_fwd', 'cuba_fwd_cfg0', 'cuba_bwd', 'li_fwd', 'li_bwd', 'alif_fwd', 'alif_bwd', 'adrf_fwd', 'adrf_bwd',
              'shift', 'fir_conv', 'delay_fir_fwd', 'delay_fir_bwd')
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

        def forward_of(y):
            for layer in net:
                y = layer(y)
            return y

        def forward():
            return forward_of(x)

        if name == 'cfg4_fwd_graph':
            # the same forward pass captured once and replayed as one CUDA graph: at a few samples per GPU
            # the eager pass is bound by the ~60 launches it makes, not by their kernels
            graphed = slayer.utils.Graphed(lambda inp: forward_of(inp), x)
            return (lambda: graphed(graphed.input)), 10, (net, x, graphed)
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
    if name.startswith(SYNAPSE):
        gen = torch.Generator(device=device).manual_seed(seed)
        x = (torch.rand(shape, device=device, generator=gen) < 0.05).float()

        def grid_weight(*wshape):   # weights on the 1/32 grid of the blocks' quantiser
            return torch.randint(-64, 64, wshape, device=device, generator=gen).float() / 32
        if name.startswith('pool_'):
            w = torch.ones(1, 1, 4, 4, 1, device=device)
            if name == 'pool_fwd':
                return (lambda: _ops.pool_fwd(x, w)), 1, (x, w)
            gy = _ops.pool_fwd(x, w)
            return (lambda: _ops.pool_bwd(gy, w, tuple(shape))), 1, (gy, w)
        if name == 'conv5_fwd':
            w = grid_weight(16, 2, 5, 5, 1)
            return (lambda: _ops.conv_fwd(x, w, (2, 2))), 1, (x, w)
        if name == 'conv3_fwd':
            w = grid_weight(32, 16, 3, 3, 1)
            return (lambda: _ops.conv_fwd(x, w, (1, 1))), 1, (x, w)
        if name == 'conv3_dgrad':
            w = grid_weight(32, 16, 3, 3, 1)
            gy = torch.empty(shape, device=device).normal_(0.0, 1.0, generator=gen)
            return (lambda: _ops.conv_dgrad(gy, w, (1, 1))), 1, (gy, w)
        if name == 'conv3_wgrad':
            gy = torch.empty((shape[0], 32) + tuple(shape[2:]), device=device).normal_(0.0, 1.0, generator=gen)
            return (lambda: _ops.conv_wgrad(x, gy, (32, 16, 3, 3, 1), (1, 1))), 2, (x, gy)
    if name == 'cuba_fwd_train':
        cd, vd = one(1024), one(123)

        def step():
            return _ops.cuba_fwd(d['x'], cd, vd, zeros, zeros, THR, W_SCALE, want_current=True, want_spike=True)
        return step, 1, d
    if name == 'cuba_bwd_dgrad':
        cd, vd = one(1024), one(123)
        r = _ops.cuba_fwd(d['x'], cd, vd, zeros, zeros, THR, W_SCALE, want_current=True, want_spike=True)
        d.update(voltage=r['voltage'], current=r['current'])
        del d['x'], r

        def step():
            return _ops.cuba_bwd(d['g'], d['voltage'], THR, d['current'], cd, vd, 125.0, 0.1, False, True)
        return step, 5, d   # the reverse scan plus two two-step folds of the decay-gradient partials
    if name == 'li_bwd_dgrad':
        dec = one(1024)
        d['x'] = torch.empty(shape, device=device).normal_(0.3, 1.0)
        d['y'] = _ops.li_fwd(d['x'], dec, zeros, W_SCALE)
        d['g'] = torch.empty(shape, device=device).normal_(0.0, 1.0)
        del d['x']

        def step():
            return _ops.li_bwd(d['g'], d['y'], dec, True)
        return step, 3, d
    if name in ('ath_fwd', 'apth_fwd'):
        d['x'] = torch.empty(shape, device=device).normal_(0.5, 1.5)
        ths = torch.ones(lead, device=device)
        if name == 'ath_fwd':
            return (lambda: _ops.ath_fwd(d['x'], zeros, one(410), ths, one(410), 0.5, 1.0, W_SCALE)), 1, d
        d['im'] = torch.empty(shape, device=device).normal_(0.0, 1.5)
        return (lambda: _ops.apth_fwd(d['x'], d['im'], zeros, zeros, one(410), ths, one(410), 0.25, 0.5, W_SCALE)), 1, d
    if name in ('res_fwd', 'res_bwd', 'res_bwd_pgrad', 'adres_fwd', 'cspike_fwd', 'cspike_bwd'):
        gen = torch.Generator(device=device).manual_seed(seed + 1)
        period = 10 + 30 * torch.rand(C, device=device, generator=gen)
        sd = (4096 * torch.sin(2 * np.pi / period) * 0.9).round()
        cdec = (4096 * torch.cos(2 * np.pi / period) * 0.9).round()
        re = torch.empty(shape, device=device).normal_(0.0, 0.5, generator=gen)
        im = torch.empty(shape, device=device).normal_(0.0, 0.5, generator=gen)
        keep = dict(re=re, im=im)
        if name == 'res_fwd':
            return (lambda: _ops.res_fwd(re, im, sd, cdec, zeros, zeros, W_SCALE)), 1, keep
        if name == 'adres_fwd':
            ths = 0.5 * torch.ones(lead, device=device)
            return (lambda: _ops.adres_fwd(re, im, sd, cdec, one(410), one(410), zeros, zeros, zeros, ths, 0.25, 0.5,
                                           W_SCALE)), 1, keep
        if name == 'cspike_fwd':
            return (lambda: _ops.cspike_fwd(re, im, 0.5, zeros, False, 1)), 1, keep
        g = torch.empty(shape, device=device).normal_(0.0, 1.0, generator=gen)
        keep['g'] = g
        if name == 'cspike_bwd':
            return (lambda: _ops.cspike_bwd(re, im, 0.5, g, 0.25, 10.0, False)), 1, keep
        # the two gradient streams are separate tensors: the same tensor twice would be read from HBM once
        g2 = torch.empty(shape, device=device).normal_(0.0, 1.0, generator=gen)
        keep['g2'] = g2
        if name == 'res_bwd':
            return (lambda: _ops.res_bwd(g, g2, None, None, sd, cdec, False)), 1, keep
        return (lambda: _ops.res_bwd(g, g2, re, im, sd, cdec, True)), 3, keep   # the scan and one fold per decay gradient
    if name in ('spike_fwd', 'spike_bwd'):
        v = torch.empty(shape, device=device).normal_(1.0, 1.0)
        if name == 'spike_fwd':
            return (lambda: _ops.spike_fwd(v, THR, False, 1)), 1, v
        g = torch.empty(shape, device=device).normal_(0.0, 1.0)
        return (lambda: _ops.spike_bwd(v, THR, g, 125.0, 0.1, False)), 1, (v, g)
    if name == 'sdnn_bwd':
        thr = one(0.1)
        r = _ops.sdnn_relu_fwd(d['x'], thr, None, None, None, None, 4096, want_act=True)
        d['act'] = r['activation']
        d['g'] = torch.empty(shape, device=device).normal_(0.0, 1.0)
        del d['x'], r

        def step():
            return _ops.sdnn_relu_bwd(d['g'], d['act'], None, thr, 1.0, 1.0, False)
        return step, 1, d
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
    if name in ('cuba_fwd_cfg0_api', 'cuba_fwd_cfg0_graph'):
        import lava_dl_b200.slayer as slayer
        neuron = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03).to(device)
        if name == 'cuba_fwd_cfg0_graph':
            graphed = slayer.utils.Graphed(neuron, d['x'])
            return (lambda: graphed(graphed.input)), 1, (d, neuron, graphed)

        def step():
            with torch.no_grad():
                return neuron(d['x'])
        return step, 1, (d, neuron)
    if name == 'cuba_fwd_infer':
        cd, vd = one(1024), one(123)

        def step():
            return _ops.cuba_fwd(d['x'], cd, vd, zeros, zeros, THR, W_SCALE, want_current=False, want_spike=True,
                                 want_voltage=False)
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
    if name in ('alif_fwd', 'alif_fwd_infer', 'alif_bwd'):
        cd, vd, td, rd = one(819), one(205), one(410), one(410)
        ths = torch.ones(lead, device=device)
        args = (d['x'], cd, vd, rd, td, zeros, zeros, zeros, ths, 0.5, 1.0, W_SCALE)
        if name in ('alif_fwd', 'alif_fwd_infer'):
            def step():
                return _ops.alif_fwd(*args, dynamics_mode=False, spikes_only=name.endswith('infer'),
                                     margin=not name.endswith('infer'))
            return step, 1, d
        (spk, margin, _), _ = _ops.alif_fwd(*args, dynamics_mode=False, margin=True)
        d.update(margin=margin)
        del d['x'], spk

        def step():
            return _ops.cuba_bwd(d['g'], d['margin'], 0.0, None, cd, vd, 100.0, 0.1, False, False)
        return step, 1, d
    if name in ('adrf_fwd', 'adrf_fwd_infer', 'adrf_bwd'):
        gen = torch.Generator(device=device).manual_seed(seed + 1)
        period = 10 + 30 * torch.rand(C, device=device, generator=gen)
        sd = (4096 * torch.sin(2 * np.pi / period) * 0.9).round()
        cdec = (4096 * torch.cos(2 * np.pi / period) * 0.9).round()
        ad = dict(ref_decay=one(410), th_decay=one(410), ref_state=zeros, th_state=0.5 * torch.ones(lead, device=device),
                  th_step=0.25, th0=0.5)
        if name in ('adrf_fwd', 'adrf_fwd_infer'):
            def step():
                return _ops.rf_fwd(d['re'], d['im'], sd, cdec, zeros, zeros, 0.5, W_SCALE, adaptive=ad,
                                   spikes_only=name.endswith('infer'), margin=not name.endswith('infer'))
            return step, 1, d
        outs, _ = _ops.rf_fwd(d['re'], d['im'], sd, cdec, zeros, zeros, 0.5, W_SCALE, adaptive=ad, margin=True)
        d.update(margin=outs[1], imag=outs[2])
        del d['re'], d['im'], outs

        def step():
            return _ops.rf_bwd(d['g'], d['margin'], d['imag'], 0.0, sd, cdec, 50.0, 0.1, False, False)
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
def _allreduce(value, op, device, dist):
    if dist is None:
        return float(value)
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=getattr(dist.ReduceOp, op))
    return float(t.item())


def host_copy_peak(nbytes, device, dist, reps=3):
    """What this host gives one rank for pinned-memory copies of one e2e chunk, in GB/s: host -> device
    alone, device -> host alone, and both at once (each direction's rate), with every rank copying at
    the same time.  The slowest rank is reported: it is the one the end-to-end step waits for."""
    n = nbytes // 4
    h_in = torch.empty(n, pin_memory=True).zero_()
    h_out = torch.empty(n, pin_memory=True)
    d_a, d_b = torch.empty(n, device=device), torch.zeros(n, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def timed(do_h2d, do_d2h):
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(s1):
            a0.record(s1)
            for _ in range(reps if do_h2d else 0):
                d_a.copy_(h_in, non_blocking=True)
            a1.record(s1)
        with torch.cuda.stream(s2):
            b0.record(s2)
            for _ in range(reps if do_d2h else 0):
                h_out.copy_(d_b, non_blocking=True)
            b1.record(s2)
        torch.cuda.synchronize(device)
        up = nbytes * reps / (a0.elapsed_time(a1) * 1e-3) / 1e9 if do_h2d else None
        down = nbytes * reps / (b0.elapsed_time(b1) * 1e-3) / 1e9 if do_d2h else None
        return up, down

    timed(True, True)  # first touch
    h2d, _ = timed(True, False)
    _, d2h = timed(False, True)
    both = timed(True, True)
    out = {'h2d': _allreduce(h2d, 'MIN', device, dist), 'd2h': _allreduce(d2h, 'MIN', device, dist),
           'h2d_while_d2h': _allreduce(both[0], 'MIN', device, dist),
           'd2h_while_h2d': _allreduce(both[1], 'MIN', device, dist), 'chunk_bytes': nbytes,
           'how': 'pinned copy_ of one chunk x%d per direction, all ranks at once, slowest rank' % reps}
    del h_in, h_out, d_a, d_b
    return out


def e2e_cuba(shape, device, steps, warmup, dist, local):
    """Host-resident input -> spikes back on the host, streamed in batch chunks through
    slayer.neuron.cuba.Neuron: three streams (H2D, compute, D2H), chunk k+1 uploads while chunk k
    computes.  Timed twice: with the fp32 spike tensor the reference API returns (forward), and with
    the opt-in bit-packed result (forward_packed), whose copy back is 32 times smaller."""
    import lava_dl_b200.slayer as slayer
    from lava_dl_b200 import _host
    B, C, T = shape
    chunk = max(1, min(B, 8))
    nchunks = (B + chunk - 1) // chunk
    place = _host.bind_near_gpu(local)  # pinned pages on the GPU's NUMA node, before they are allocated
    try:
        x_host = torch.empty(shape, pin_memory=True)
        s_host = torch.empty(shape, pin_memory=True)
        b_host = torch.empty((B, C, (T + 31) // 32), dtype=torch.int32, pin_memory=True)
    except RuntimeError:
        _host.restore_affinity(place)
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

    def one_pass(packed):
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
                res = neuron.forward_packed(xbuf[i][:b1 - b0]) if packed else neuron(xbuf[i][:b1 - b0])
            free_x[i].record(comp)
            done = torch.cuda.Event()
            done.record(comp)
            with torch.cuda.stream(down):
                down.wait_event(done)
                (b_host if packed else s_host)[b0:b1].copy_(res, non_blocking=True)
                res.record_stream(down)
            outs.append(res)
        comp.wait_stream(down)
        return outs

    def timed(packed):
        for e in free_x:
            e.record(comp)
        for _ in range(max(1, warmup)):
            one_pass(packed)
        torch.cuda.synchronize(device)
        if dist is not None:
            dist.barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record(comp)
        for _ in range(steps):
            one_pass(packed)
        t1.record(comp)
        torch.cuda.synchronize(device)
        return _allreduce(t0.elapsed_time(t1) / steps, 'MAX', device, dist)

    ms = timed(False)
    rate = float(s_host[:chunk].mean())
    ms_packed = timed(True)
    from lava_dl_b200 import _ops
    same = bool(torch.equal(_ops.unpack_spikes(b_host[:1], T), s_host[:1]))
    nbytes = int(np.prod(shape)) * 4
    del xbuf, x_host, s_host
    peak = host_copy_peak(chunk * C * T * 4, device, dist)
    _host.restore_affinity(place)
    return {'ms': ms, 'h2d': nbytes, 'd2h': nbytes, 'launches': nchunks, 'rate': rate, 'ms_packed': ms_packed,
            'd2h_packed': int(b_host.numel()) * 4, 'packed_equals_fp32': same, 'host_copy_peak_GBps': peak,
            'placement': {k: place[k] for k in ('node', 'mempolicy')} | {'cpus_bound': place['cpus'] is not None}}


def fwd_bwd_cuba(shape, device, steps, warmup, dist):
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
    if dist is not None:
        dist.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        one_step()
    t1.record()
    torch.cuda.synchronize(device)
    ms = _allreduce(t0.elapsed_time(t1) / steps, 'MAX', device, dist)
    parity = parity_cuba_grad(x, neuron)
    return ms, n_reduced, parity


# ---------------------------------------------------------------------------
# parity of what was timed (outside the timed regions)
# ---------------------------------------------------------------------------
PARITY_SAMPLES = 1   # samples of the batch replayed through the CPU oracle


def parity_cuba_fwd(x, out):
    """The last timed output against the oracle on the same input, first samples of the batch."""
    from oracle import oracle as O
    O.set_threads(os.cpu_count() or 1)
    n = min(PARITY_SAMPLES, x.shape[0])
    want = O.cuba(x[:n].cpu().numpy(), 1.25, 1024.0, 123.0)
    spike = out['spike'][:n].cpu().numpy()
    voltage = out['voltage'][:n].cpu().numpy()
    return {'spikes_exact': bool(np.array_equal(spike, want['spike'])),
            'voltage_exact': bool(np.array_equal(voltage, want['voltage'])),
            'rows_checked': int(n * x.shape[1]), 'steps_per_row': int(x.shape[-1]),
            'spikes_in_checked_rows': int(want['spike'].sum()), 'against': 'CPU oracle, same input bits'}


def parity_cuba_grad(x, neuron):
    """grad_x of the last training step (loss = sum of spikes) against the oracle: 1e-5 of the sum of
    the magnitudes each element adds up, and the share that also meets 1e-5 element-wise."""
    from oracle import oracle as O
    O.set_threads(os.cpu_count() or 1)
    n = min(PARITY_SAMPLES, x.shape[0])
    xs = x[:n].detach().cpu().numpy()
    cd = neuron.current_decay.detach().cpu().numpy()
    vd = neuron.voltage_decay.detach().cpu().numpy()
    ones = np.ones_like(xs)
    want = O.cuba(xs, 1.25, cd, vd, grad_spike=ones)
    got = x.grad[:n].cpu().numpy().astype(np.float64)
    ref = want['grad_x'].astype(np.float64)
    scale = np.maximum(O.cuba_grad_x_scale(want['voltage'], 1.25, ones, cd, vd), 1e-2 * np.abs(ref).max())
    err = np.abs(got - ref)
    return {'grad_x_within_1e-5_of_term_magnitudes': bool(np.all(err <= 1e-5 * scale)),
            'grad_x_share_within_1e-5_elementwise': float(np.mean(err <= 1e-5 * np.abs(ref))),
            'rows_checked': int(n * x.shape[1]), 'against': 'CPU oracle, same input bits'}


# ---------------------------------------------------------------------------
# timing of one workload
# ---------------------------------------------------------------------------
def time_steps(step, steps, warmup, device, dist, sampler=None):
    """W untimed steps, then K steps bracketed by barrier + synchronize, CUDA events on the
    launching stream; returns (ms per step as the max over ranks, per-step times of this rank)."""
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(warmup):
        step()
    barrier()
    stream = torch.cuda.current_stream(device)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]

    def run():
        barrier()
        evs[0].record(stream)
        for i in range(steps):
            step()
            evs[i + 1].record(stream)
        barrier()

    if sampler is None:
        run()
    else:
        with sampler:
            run()
    total_ms = _allreduce(evs[0].elapsed_time(evs[-1]), 'MAX', device, dist)
    return total_ms / steps, [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]


# legs reported beside the headline in the default run: every benchmark configuration's kernels
EXTRA_LEGS = ('cuba_fwd_infer', 'cuba_bwd', 'alif_fwd', 'alif_fwd_infer', 'alif_bwd', 'adrf_fwd', 'adrf_fwd_infer', 'adrf_bwd', 'shift', 'fir_conv', 'delay_fir_fwd',
              'delay_fir_bwd', 'cuba_fwd_cfg0', 'cuba_fwd_cfg0_api', 'cuba_fwd_cfg0_graph', 'cfg4_fwd', 'cfg4_fwd_graph', 'cfg4_train')


def run_extra_legs(device, dist, world, rank, steps=5, warmup=3, legs=EXTRA_LEGS):
    """{name: {shape, ms, GB/s, frac}} for the other kernels of the path (full benchmark shapes, one
    shard per GPU) and for the conv network, whose global batch of 32 is split over the ranks
    (strong scaling, one flattened all-reduce of weight and decay gradients per training step)."""
    peak, _ = peaks()
    out = {}
    for name in legs:
        wl = WORKLOADS[name]
        shape = tuple(wl.shape)
        net = name.startswith(NETWORKS)
        if net and world > 1:
            shape = (max(1, shape[0] // world),) + shape[1:]
        step, launches, keep = build_step(name, shape, device, seed=99 + rank)
        ms, per = time_steps(step, steps, warmup, device, dist)
        units = wl.units(shape)
        leg = {'shape': list(shape), 'ms': ms}
        if net:
            leg['value'] = units * world / (ms * 1e-3)
            leg['unit'] = wl.unit
            leg['global_batch'] = shape[0] * world
            leg['scaling'] = 'strong'
            if name == 'cfg4_train':
                nparam = sum(q.numel() for q in keep[0].parameters() if q.requires_grad)
                leg['allreduce_bytes_per_step'] = 4 * nparam if world > 1 else 0
        else:
            gbs = wl.bytes(shape) / (statistics.mean(per) * 1e-3) / 1e9
            leg.update({'GBps': gbs, 'frac': gbs / peak, 'bytes_per_unit': wl.bpu})
        out[name] = leg
        del step, keep
        torch.cuda.empty_cache()
    return out


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
    ap.add_argument('--no-extra', action='store_true', help='skip the per-configuration legs of the default run')
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
        if wl.name not in CPU_PORTED:
            print(json.dumps({'impl': 'reference', 'unavailable': 'the CPU oracle is not timed on this workload'}))
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
        import datetime
        import torch.distributed as dist
        # a rank that dies between steps must end the others' next collective with an error, not a hang
        dist.init_process_group('nccl', device_id=device, timeout=datetime.timedelta(seconds=300))

    net = wl.name.startswith(NETWORKS)
    if net and world > 1:
        shape = (max(1, shape[0] // world),) + shape[1:]   # the networks split one global batch
    step, launches_per_step, keep = build_step(wl.name, shape, device, seed=1234 + rank)
    units = wl.units(shape)
    clocks = ClockSampler(local)
    ms_per_step, per = time_steps(step, args.steps, args.warmup, device, dist, sampler=clocks)
    value = units * world / (ms_per_step * 1e-3)

    parity = None
    if wl.name == 'cuba_fwd':
        parity = parity_cuba_fwd(keep['x'], step())
        if dist is not None:
            ok = _allreduce(float(parity['spikes_exact'] and parity['voltage_exact']), 'MIN', device, dist)
            parity['all_ranks_exact'] = bool(ok)

    peak, peak_kind = peaks()
    kern_ms = statistics.mean(per)   # a step is one kernel (plus, with parameter gradients, two tiny fold kernels)
    achieved = wl.bytes(shape) / (kern_ms * 1e-3) / 1e9
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
        'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'strong' if net else 'weak',
        'vs_baseline': None,
        'dtype': 'f32 (3xTF32 products, fp32 accumulate)' if 'fir' in wl.name else 'int32+f32', 'data': 'synthetic',
        'config': {'workload': f'{wl.name} {list(shape)} per GPU', 'global_batch': shape[0] * world,
                   'l2': 'inputs larger than L2 (no flush)',
                   'parallelism': f'batch shards x{world}, no forward collective'},
        'gpu_launches': args.steps * launches_per_step,
        'roofline': roofline,
        'clocks': clocks.summary(),
    }
    if parity is not None:
        line['parity'] = parity

    del keep, step
    torch.cuda.empty_cache()

    default_run = wl.name == 'cuba_fwd' and args.batch == 0
    if wl.name == 'cuba_fwd' and not args.no_e2e:
        r = e2e_cuba(shape, device, steps=max(2, min(args.steps, 5)), warmup=1, dist=dist, local=local)
        if r is not None:
            pk = r['host_copy_peak_GBps']
            # the step moves the batch up and the result down at once: the ceiling is the slower direction
            ceil_ms = max(r['h2d'] / (pk['h2d_while_d2h'] * 1e9), r['d2h'] / (pk['d2h_while_h2d'] * 1e9)) * 1e3
            ceil_ms_packed = r['h2d'] / (pk['h2d'] * 1e9) * 1e3
            line['e2e'] = {
                'value': units * world / (r['ms'] * 1e-3), 'unit': wl.unit, 'h2d_bytes_per_step': r['h2d'],
                'd2h_bytes_per_step': r['d2h'], 'ms_per_step': r['ms'],
                'path': 'slayer.neuron.cuba.Neuron.forward on pinned host batches, chunked over batch',
                'spike_rate': r['rate'], 'host_copy_peak_GBps': pk, 'placement': r['placement'],
                'frac_of_host_copy_peak': ceil_ms / r['ms'],
                'packed': {'value': units * world / (r['ms_packed'] * 1e-3), 'ms_per_step': r['ms_packed'],
                           'd2h_bytes_per_step': r['d2h_packed'], 'equals_fp32_result': r['packed_equals_fp32'],
                           'frac_of_host_copy_peak': ceil_ms_packed / r['ms_packed'],
                           'path': 'Neuron.forward_packed: same spikes as 32-step bit words (opt-in)'}}
    if wl.name == 'cuba_fwd' and not args.no_e2e:
        ms, n_red, gpar = fwd_bwd_cuba(shape, device, steps=max(2, min(args.steps, 5)), warmup=2, dist=dist)
        # bytes: fwd x in, spike + voltage + current out (16); ones-like grad written + read (8);
        # bwd g_spike, voltage, current in, g_x out (16)
        line['fwd_bwd'] = {'value': units * world / (ms * 1e-3), 'unit': wl.unit, 'ms_per_step': ms,
                           'allreduce_elements': n_red, 'parity': gpar,
                           'path': 'cuba.Neuron(requires_grad=True)(x).sum().backward() + one all-reduce of decay grads'}
        torch.cuda.empty_cache()
    if default_run and not args.no_extra:
        line['extra'] = run_extra_legs(device, dist, world, rank)
    if wl.name.startswith('recurrent'):
        line['roofline'] = None  # latency-bound walk over time plus two GEMMs
        line['config']['network'] = 'block.cuba.Recurrent(512, 512), spikes in at 5 %'
    if wl.name.startswith('cfg4'):
        line['roofline'] = None  # a chain of synapse and neuron kernels has no single roof
        line['config']['network'] = 'Pool4-Conv(2,16,5)-Pool2-Conv(16,32,3)-Pool2-Flatten-Dense(2048,512)-Dense(512,11), CUBA'
        line['config']['parallelism'] = f'global batch {shape[0] * world} split over {world} GPUs, one all-reduce of weight gradients'
    if rank == 0 and not args.no_cpu and wl.name in CPU_PORTED:
        cpu, _ = time_cpu(wl, steps=3, warmup=1)
        # context, not measured here: lava-dl's own Python loops ran this neuron at about 1e7
        # neuron-steps/s on 8 host threads when the path was surveyed (two orders below the C port)
        cpu['reference_python_context'] = '~1.0e7 neuron-steps/s (lava-dl CPU path, 8 threads, other host; not timed in this run)'
        line['cpu_baseline'] = cpu
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == '__main__':
    main()
