"""A small CUBA conv network assembled from the block mirror, against the same
network built from lava-dl's own blocks (tests/golden/network_cuba_conv.npz).

Synaptic weights are quantised to multiples of 1/32 and the inputs of every
synapse are 0/1 spikes, so every dendritic sum is exactly representable whatever
the convolution algorithm or summation order: cuDNN on the GPU and the
reference's CPU convolution feed identical values to the neurons, and the spike
tensors of all eight layers must match bit for bit.  Gradients pass through
cuDNN's backward kernels, whose summation order differs from the CPU's; they are
compared with a relative L2 criterion (1e-4) instead of element-wise.  The decay
gradients of the early layers are sums of ~10^5 signed products that cancel to
values orders of magnitude below the products themselves (5e-13 in layer 0);
they get 5e-3 here, while test_gpu_parity.py holds the same sums to 1e-5 of
their term magnitudes on the kernels in isolation."""

import numpy as np
import pytest
import torch

from _util import assert_exact, load_golden

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a = a.detach().cpu().numpy().astype(np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def build(slayer, cuda):
    p = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03, requires_grad=True)
    blk = slayer.block.cuba
    return torch.nn.ModuleList([
        blk.Pool(p, 4), blk.Conv(p, 2, 16, 5, padding=2, weight_scale=4), blk.Pool(p, 2),
        blk.Conv(p, 16, 32, 3, padding=1, weight_scale=3), blk.Pool(p, 2), blk.Flatten(),
        blk.Dense(p, 128, 64, weight_scale=3), blk.Dense(p, 64, 11, weight_scale=3, delay=True),
    ]).to(cuda)


def test_network_matches_reference_blocks(cuda):
    import lava_dl_b200.slayer as slayer
    g = load_golden('network_cuba_conv')
    net = build(slayer, cuda)
    x = torch.tensor(g['x'], device=cuda)
    with torch.no_grad():
        y = x
        for layer in net:  # binds shapes and creates the delay parameter
            y = layer(y)
        for i, layer in enumerate(net):
            if hasattr(layer, 'synapse'):
                layer.synapse.weight.data = torch.tensor(g[f'weight{i}'], device=cuda)
        net[7].delay.delay.data = torch.tensor(g['delay'], device=cuda)

    xin = x.clone().requires_grad_(True)
    y = xin
    for i, layer in enumerate(net):
        y = layer(y)
        assert_exact(y, g[f'act{i}'], f'layer {i} output')
    (y * torch.tensor(g['grad_out'], device=cuda)).sum().backward()

    assert rel_l2(xin.grad, g['grad_x']) < 1e-4
    for i, layer in enumerate(net):
        if f'grad_weight{i}' in g:
            assert rel_l2(layer.synapse.weight.grad, g[f'grad_weight{i}']) < 1e-4, f'weight grad of layer {i}'
        if hasattr(layer, 'neuron'):
            for k in ('current_decay', 'voltage_decay'):
                assert rel_l2(getattr(layer.neuron, k).grad, g[f'grad_{k}{i}']) < 5e-3, f'{k} grad of layer {i}'
    assert rel_l2(net[7].delay.delay.grad, g['grad_delay']) < 1e-4


def test_count_log_and_persistent_step_delay(cuda):
    import lava_dl_b200.slayer as slayer
    p = dict(threshold=1.0, current_decay=0.5, voltage_decay=0.1, persistent_state=True)
    block = slayer.block.cuba.Dense(p, 6, 4, weight_scale=8, count_log=True).to(cuda)
    gen = torch.Generator().manual_seed(3)
    x = (torch.rand(2, 6, 64, generator=gen) < 0.3).float().to(cuda)
    with torch.no_grad():
        full, rate = block(x)
        assert 0 <= float(rate) <= 1 and abs(float(rate) - float((full > 0).float().mean())) < 1e-7
        for name, buf in block.neuron.named_buffers():
            if name.endswith('_state'):
                buf.zero_()
        block.delay_buffer = None
        a, _ = block(x[..., :30].contiguous())
        b, _ = block(x[..., 30:].contiguous())
    assert_exact(torch.cat([a, b], dim=-1), full, 'chunked run with carried state and delay buffer')


@pytest.mark.parametrize('shape,k', [((2, 3, 8, 8, 40), 2), ((1, 2, 5, 7, 12), 2), ((2, 1, 6, 9, 33), 4),
                                     ((1, 1, 12, 12, 7), (3, 2)), ((2, 2, 4, 4, 1), 4)])
def test_sum_pool_kernel_matches_conv3d(shape, k, cuda):
    """The gather-and-add pooling kernel against the Conv3d formulation it replaces
    (same module, fall-back path), forward and backward, odd sizes included.  (Sizes
    whose padded height is still not a multiple of the window make the reference's
    own reshape fail, synapse/layer.py:493-507, so they are not comparable.)"""
    import lava_dl_b200.slayer as slayer
    gen = torch.Generator().manual_seed(sum(shape))
    pool = slayer.synapse.Pool(k, weight_scale=2).to(cuda)
    with torch.no_grad():  # non-uniform multiples of 1/32 so every sum is exact in fp32
        pool.weight.copy_(torch.randint(-64, 64, pool.weight.shape, generator=gen).float().to(cuda) / 32)
    x = (torch.rand(shape, generator=gen) < 0.3).float().to(cuda)
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    fast = pool(xa)
    assert fast.grad_fn is not None and 'SumPool' in type(fast.grad_fn).__name__
    pool.padding = (0, 0, 0)
    pool.weight.requires_grad_(True)  # makes forward() take the Conv3d path
    slow = pool(xb)
    pool.weight.requires_grad_(False)
    assert 'SumPool' not in type(slow.grad_fn).__name__
    assert_exact(fast, slow, 'pooled sums')
    g = torch.randint(-8, 8, fast.shape, generator=gen).float().to(cuda) / 4
    fast.backward(g)
    slow.backward(g)
    assert_exact(xa.grad, xb.grad, 'pool input gradient')


@pytest.mark.parametrize('shape,co,k,pad', [((2, 2, 8, 8, 40), 16, 5, 2), ((1, 3, 7, 9, 12), 5, 3, 1),
                                            ((2, 16, 6, 6, 33), 32, 3, 1), ((1, 4, 5, 6, 8), 20, (3, 1), (0, 0)),
                                            ((3, 1, 4, 4, 1), 2, 1, 0),
                                            # forward fits the kernel, the swapped (input-gradient) problem does not:
                                            # 200 output channels x 9 taps of weights, and N * H = 66000 rows
                                            ((1, 4, 6, 6, 8), 200, 3, 1), ((2200, 1, 30, 3, 4), 2, (3, 1), (0, 0)),
                                            # tensor-core shapes: two chunks of input channels; 5 x 5 with a ragged
                                            # last time chunk; two groups of output channels with a partial one and
                                            # a width that is no multiple of four; 1 x 1; a partial channel chunk
                                            ((2, 16, 6, 6, 64), 32, 3, 1), ((1, 2, 9, 10, 44), 16, 5, 2),
                                            ((2, 16, 5, 7, 32), 70, 3, 1), ((2, 24, 3, 5, 96), 24, 1, 0),
                                            ((1, 11, 4, 9, 36), 5, 3, 0), ((3, 3, 12, 12, 300), 8, 5, 1),
                                            # few input channels packed 2 or 4 to a column: one channel 5 x 5, three channels 1 x 1
                                            # and 3 x 3 (an MMA's eight rows then span several taps, or several output columns)
                                            ((2, 1, 6, 7, 36), 8, 5, 2), ((2, 3, 5, 6, 64), 8, 1, 0), ((2, 4, 6, 7, 36), 8, 3, 0),
                                            # rows with more (column, time word) positions than the weight-gradient kernel has
                                            # threads; a row too wide for its shared memory (ATen takes that gradient)
                                            ((1, 1, 4, 100, 8), 8, 3, 1), ((1, 2, 4, 260, 8), 16, 5, 2),
                                            # wide layers: the tensor-core kernel takes the input channels in blocks (three launches
                                            # of 16, 16 and 8 channels; the input gradient of the second in two of 16)
                                            ((2, 40, 6, 6, 64), 32, 3, 1), ((2, 16, 6, 9, 32), 32, 3, 1)])
def test_conv_kernel_matches_conv3d(shape, co, k, pad, cuda):
    """The direct convolution synapse kernel against F.conv3d: exact on spikes with
    weights on the 1/32 grid (every partial sum is representable), 1e-5 on floats;
    backward (own kernels where the shape allows, else ATen) against autograd of conv3d and float64."""
    import torch.nn.functional as F
    import lava_dl_b200.slayer as slayer
    from _util import assert_close
    gen = torch.Generator().manual_seed(sum(shape) + co)
    conv = slayer.synapse.Conv(shape[1], co, k, padding=pad).to(cuda)
    with torch.no_grad():
        conv.weight.copy_(torch.randint(-128, 127, conv.weight.shape, generator=gen).float().to(cuda) / 32)
    x = (torch.rand(shape, generator=gen) < 0.3).float().to(cuda)
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    fast = conv(xa)
    assert 'SpikeConv' in type(fast.grad_fn).__name__
    from lava_dl_b200 import _native, _ops
    geo = (shape[0], shape[1], co, shape[2], shape[3], *conv.kernel_size[:2], *conv.padding[:2], shape[-1])
    fits = _native.load().sb_conv_fits_tensor_cores(*geo) == 1
    assert fits == (shape[-1] % 4 == 0 and shape[-1] >= 32)
    if fits:
        # both kernels on the same spikes: identical sums
        w = conv._hooked_weight()
        assert_exact(_ops.conv_fwd(x, w, conv.padding, path=1), _ops.conv_fwd(x, w, conv.padding, path=-1),
                     'tensor-core kernel against the automatic choice')
    slow = F.conv3d(xb, conv.weight, None, conv.stride, conv.padding, conv.dilation, conv.groups)
    assert_exact(fast, slow, 'convolution of spikes')
    g = torch.randint(-8, 8, fast.shape, generator=gen).float().to(cuda) / 4
    w_fast = torch.autograd.grad(fast, [xa, conv.weight], g)
    w_slow = torch.autograd.grad(slow, [xb, conv.weight], g)
    assert rel_l2(w_fast[0], w_slow[0].cpu().numpy()) < 1e-6 and rel_l2(w_fast[1], w_slow[1].cpu().numpy()) < 1e-6
    xf = torch.randn(shape, generator=gen).to(cuda)
    with torch.backends.cudnn.flags(allow_tf32=False):
        want = F.conv3d(xf, conv.weight, None, conv.stride, conv.padding)
    # float operands: 1e-5 of the sum of the term magnitudes (the tensor-core path adds three TF32
    # products per term, each within 2^-21 of the term; plain relative error where nothing cancels)
    with torch.backends.cudnn.flags(allow_tf32=False):
        mag = F.conv3d(xf.abs(), conv.weight.detach().abs(), None, conv.stride, conv.padding)
    assert_close(conv(xf), want, 'convolution of floats', scale=mag.cpu().numpy())
    if fits:
        assert_close(_ops.conv_fwd(xf, conv._hooked_weight(), conv.padding, path=1), want,
                     'convolution of floats, tensor cores', scale=mag.cpu().numpy())
        wf = torch.randn(conv.weight.shape, generator=gen).to(cuda)   # weights off the TF32 grid as well
        with torch.backends.cudnn.flags(allow_tf32=False):
            want2 = F.conv3d(xf, wf, None, conv.stride, conv.padding)
            mag2 = F.conv3d(xf.abs(), wf.abs(), None, conv.stride, conv.padding)
        assert_close(_ops.conv_fwd(xf, wf, conv.padding, path=1), want2,
                     'convolution of floats with float weights, tensor cores', scale=mag2.cpu().numpy())
    # gradients on float data against float64 on the CPU: 1e-5 of the sum of the term magnitudes
    xd = xf.double().cpu().requires_grad_(True)
    wd = conv.weight.detach().double().cpu().requires_grad_(True)
    gd = torch.randn(want.shape, generator=gen, dtype=torch.float64)
    F.conv3d(xd, wd, None, conv.stride, conv.padding).backward(gd)
    mx = xf.double().cpu().abs().requires_grad_(True)
    mw = conv.weight.detach().double().cpu().abs().requires_grad_(True)
    F.conv3d(mx, mw, None, conv.stride, conv.padding).backward(gd.abs())
    xg = xf.clone().requires_grad_(True)
    with torch.backends.cudnn.flags(allow_tf32=False):   # shapes that fall back to ATen: no TF32 there either
        gx, gw = torch.autograd.grad(conv(xg), [xg, conv.weight], gd.float().to(cuda))
    assert_close(gx, xd.grad.numpy(), 'input gradient of floats', scale=mx.grad.numpy() + 1e-30)
    assert_close(gw, wd.grad.numpy(), 'weight gradient of floats', scale=mw.grad.numpy() + 1e-30)


@pytest.mark.parametrize('shape,co,k,pad', [((3, 16, 9, 10, 64), 32, 3, 1), ((2, 2, 12, 9, 96), 16, 5, 2)])
def test_conv_tensor_cores_with_spike_rows_and_float_rows_mixed(shape, co, k, pad, cuda):
    """Input rows of spikes (exact in TF32: no lo slot) interleaved with rows of floats (split into hi + lo,
    each taking the next lo slot of the ring): the tensor-core kernel against the fp32 kernel, exact where a
    whole receptive field is spikes, 1e-5 of the term magnitudes elsewhere."""
    import torch.nn.functional as F
    from lava_dl_b200 import _ops
    from _util import assert_close
    gen = torch.Generator().manual_seed(11 + sum(shape))
    x = (torch.rand(shape, generator=gen) < 0.3).float()
    floats = torch.randn(shape, generator=gen)
    # image rows 1, 2 and 5 of every sample, and every row of the last sample's even channels, hold floats
    mask = torch.zeros(shape, dtype=torch.bool)
    mask[:, :, [1, 2, 5]] = True
    mask[-1, ::2] = True
    x = torch.where(mask, floats, x).to(cuda)
    w = (torch.randint(-128, 127, (co, shape[1], k, k, 1), generator=gen).float() / 32).to(cuda)
    tc = _ops.conv_fwd(x, w, (pad, pad), path=1)
    ref = _ops.conv_fwd(x, w, (pad, pad), path=0)
    mag = _ops.conv_fwd(x.abs(), w.abs(), (pad, pad), path=0)
    assert_close(tc, ref, 'mixed rows, tensor cores against fp32 kernel', scale=mag.cpu().numpy() + 1e-30)
    # output rows whose receptive field holds no float row: identical sums (sample 0: input rows 0 and 3, 4, 6..)
    touched = F.max_pool3d(mask.float().amax(1, keepdim=True), (k, k, 1), 1, (pad, pad, 0)).to(cuda) > 0
    clean = ~touched.expand_as(tc)
    assert clean.any()
    assert torch.equal(tc[clean], ref[clean])


def test_block_axon_delay_fused_matches_unfused(cuda):
    """A CUBA dense block with a bounded axonal delay writes step delay and axonal
    delay inside the neuron kernel; an unbounded delay takes the separate shift.
    Same spikes, same gradients (input, weights, delays), also across two calls of
    a persistent-state block."""
    import lava_dl_b200.slayer as slayer
    torch.manual_seed(7)
    params = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03, requires_grad=True, persistent_state=True)
    fused = slayer.block.cuba.Dense(params, 24, 40, delay=True, delay_shift=True).to(cuda)
    plain = slayer.block.cuba.Dense(params, 24, 40, delay=True, delay_shift=True).to(cuda)
    plain.load_state_dict(fused.state_dict(), strict=False)
    fused.delay.max_delay = 62      # bounded: fused into the neuron kernel
    plain.delay.max_delay = None    # unbounded: separate shift kernel
    x1 = (torch.rand(3, 24, 96, device=cuda) < 0.3).float()
    x2 = (torch.rand(3, 24, 96, device=cuda) < 0.3).float()
    delays = torch.rand(40, device=cuda) * 62
    for blk in (fused, plain):
        blk.delay.delay.data = delays.clone()
        blk.delay.init = True
    outs = []
    for blk in (fused, plain):
        xa = x1.clone().requires_grad_()
        ya = blk(xa)
        yb = blk(x2)                      # second call: state and delay buffer carried over
        w = torch.linspace(0.5, 1.5, ya.numel(), device=cuda).reshape(ya.shape)
        (ya * w).sum().backward()
        outs.append((ya.detach(), yb.detach(), xa.grad, blk.synapse.weight.grad.clone(), blk.delay.delay.grad.clone(),
                     blk.neuron.current_decay.grad.clone()))
    names = ('first call', 'second call', 'grad input', 'grad weight', 'grad delay', 'grad decay')
    for n, a, b in zip(names, outs[0], outs[1]):
        if n.endswith('call'):
            assert torch.equal(a, b), n
        else:
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-5 * float(b.abs().max())), n   # same kernels, same order
    assert outs[0][0].sum() > 0
