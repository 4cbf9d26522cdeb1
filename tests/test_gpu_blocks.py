"""Blocks of every neuron family and the per-time-step callers (recurrent, winner-takes-all)
against the same modules of lava-dl (tests/golden/block_*.npz, network_rf.npz, network_adrf.npz).
Spikes must match bit for bit, layer by layer; gradients pass through sums whose order differs
between the two implementations and are compared with a relative L2 criterion."""

import numpy as np
import pytest
import torch

from _util import assert_close, assert_exact, load_golden

pytestmark = pytest.mark.gpu

ALIF_P = dict(threshold=1.0, threshold_step=0.5, current_decay=0.2, voltage_decay=0.05, threshold_decay=0.1,
              refractory_decay=0.1, requires_grad=True)
CUBA_P = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03, requires_grad=True)


@pytest.fixture(scope='module')
def slayer(cuda):
    import lava_dl_b200.slayer as slayer
    return slayer


def rel_l2(a, b):
    a = a.detach().cpu().numpy().astype(np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def T(a, cuda):
    return torch.tensor(a, device=cuda)


def test_alif_recurrent_block(cuda, slayer):
    """The walk over time with a neuron the one-launch kernel does not cover: step by step, as the
    reference does it; two calls (the neuron state persists) and one backward."""
    g = load_golden('block_alif_recurrent')
    rec = slayer.block.alif.Recurrent(dict(ALIF_P), 12, 20, weight_scale=3).to(cuda)
    rec.input_synapse.weight.data = T(g['weight_in'], cuda)
    rec.recurrent_synapse.weight.data = T(g['weight_rec'], cuda)
    x = T(g['x'], cuda).requires_grad_(True)
    y1 = rec(x)
    assert_exact(y1, g['out1'], 'first call')
    (y1 * T(g['grad_out'], cuda)).sum().backward()
    assert rel_l2(x.grad, g['grad_x']) < 1e-5
    assert rel_l2(rec.input_synapse.weight.grad, g['grad_weight_in']) < 1e-5
    assert rel_l2(rec.recurrent_synapse.weight.grad, g['grad_weight_rec']) < 1e-5
    with torch.no_grad():
        assert_exact(rec(T(g['x'], cuda)), g['out2'], 'second call on the kept state')


@pytest.mark.parametrize('family,params,name', [('cuba', CUBA_P, 'block_cuba_kwta'), ('alif', ALIF_P, 'block_alif_kwta')])
def test_kwta_block(family, params, name, cuda, slayer):
    """Winner-takes-all: CUBA runs the one-launch recurrent kernel with the lateral matrix and bias,
    ALIF the step-by-step walk; the learnable self excitation gets its gradient through the matrix."""
    g = load_golden(name)
    kw = getattr(slayer.block, family).KWTA(dict(params), 10, 16, 3, self_excitation=0.4, weight_scale=4,
                                            delay_shift=False).to(cuda)
    kw.synapse.weight.data = T(g['weight'], cuda)
    x = T(g['x'], cuda).requires_grad_(True)
    y1 = kw(x)
    assert_exact(y1, g['out1'], 'first call')
    (y1 * T(g['grad_out'], cuda)).sum().backward()
    assert rel_l2(x.grad, g['grad_x']) < 1e-5
    assert rel_l2(kw.synapse.weight.grad, g['grad_weight']) < 1e-5
    assert rel_l2(kw.self_excitation.grad, g['grad_self_excitation']) < 1e-4
    with torch.no_grad():
        assert_exact(kw(T(g['x'], cuda)), g['out2'], 'second call on the kept state')
    # with the one-step delay (the reference cannot differentiate that variant; forward only)
    kd = getattr(slayer.block, family).KWTA(dict(params), 10, 16, 3, self_excitation=0.4, weight_scale=4).to(cuda)
    kd.synapse.weight.data = T(g['weight'], cuda)
    with torch.no_grad():
        yd = kd(T(g['x'], cuda))
    want = np.concatenate([np.zeros_like(g['out1'][..., :1]), g['out1'][..., :-1]], axis=-1)
    assert_exact(yd, want, 'delayed by one step')


@pytest.mark.parametrize('family,name', [('rf', 'network_rf'), ('adrf', 'network_adrf')])
def test_resonator_network(family, name, cuda, slayer):
    """Conv -> Pool -> Flatten -> Dense (with axonal delay) -> Average of a resonate-and-fire family,
    complex synapses throughout."""
    g = load_golden(name)
    fam = getattr(slayer.block, family)
    if family == 'rf':
        p = dict(threshold=0.5, period=7, decay=0.1, requires_grad=True)
    else:
        p = dict(threshold=0.5, threshold_step=0.25, period=7, decay=0.1, threshold_decay=0.1,
                 refractory_decay=0.1, requires_grad=True)
    net = torch.nn.ModuleList([fam.Conv(dict(p), 2, 4, 3, padding=1, weight_scale=3), fam.Pool(dict(p), 2, weight_scale=2),
                               fam.Flatten(), fam.Dense(dict(p), 4 * 3 * 3, 10, weight_scale=4, delay=True),
                               fam.Average(5)]).to(cuda)
    x = T(g['x'], cuda)
    with torch.no_grad():
        y = x
        for layer in net:   # binds shapes and creates the delay parameter
            y = layer(y)
        for i in (0, 1, 3):
            net[i].synapse.real.weight.data = T(g[f'weight{i}_real'], cuda)
            net[i].synapse.imag.weight.data = T(g[f'weight{i}_imag'], cuda)
            assert_close(net[i].neuron.sin_decay, g[f'sin_decay{i}'], 'sin decay')
            assert_close(net[i].neuron.cos_decay, g[f'cos_decay{i}'], 'cos decay')
        net[3].delay.delay.data = T(g['delay'], cuda)
    xin = x.clone().requires_grad_(True)
    y = xin
    for i, layer in enumerate(net):
        y = layer(y)
        if i < 4:
            assert_exact(y, g[f'act{i}'], f'layer {i} output')
        else:
            assert_close(y, g[f'act{i}'], 'population average')
    (y * T(g['grad_out'], cuda)).sum().backward()
    # four layers of surrogate exponentials (evaluated as exp2 here) and cancelling rotation scans: 1e-3
    assert rel_l2(xin.grad, g['grad_x']) < 1e-3
    for i in (0, 3):
        for part in ('real', 'imag'):
            got = getattr(net[i].synapse, part).weight.grad
            assert rel_l2(got, g[f'grad_weight{i}_{part}']) < 1e-3, (i, part)


def test_recurrent_and_kwta_of_a_complex_family_fail_as_in_the_reference(cuda, slayer):
    p = dict(threshold=0.5, period=7, decay=0.1)
    x = torch.zeros(1, 4, 8, device=cuda)
    with pytest.raises(AttributeError):
        slayer.block.rf.Recurrent(dict(p), 4, 6).to(cuda)(x)
    with pytest.raises(TypeError):
        slayer.block.rf.KWTA(dict(p), 4, 6, 2).to(cuda)(x)


def test_cuba_input_block(cuda, slayer):
    g = load_golden('block_cuba_input')
    inp = slayer.block.cuba.Input(dict(CUBA_P), weight=1.5, bias=0.2).to(cuda)
    x = T(g['x'], cuda).requires_grad_(True)
    y = inp(x)
    assert_exact(y, g['out'], 'input block spikes')
    (y * T(g['grad_out'], cuda)).sum().backward()
    assert rel_l2(x.grad, g['grad_x']) < 1e-5
    assert rel_l2(inp.weight.grad, g['grad_weight']) < 1e-4
    assert rel_l2(inp.bias.grad, g['grad_bias']) < 1e-4


def test_sigma_delta_output_block(cuda, slayer):
    g = load_golden('block_sdnn_output')
    out = slayer.block.sigma_delta.Output(dict(threshold=0.1, activation=torch.nn.functional.relu, tau_grad=0.5,
                                               scale_grad=1.0, requires_grad=False), 9, 4, weight_scale=3).to(cuda)
    out.synapse.weight.data = T(g['weight'], cuda)
    with torch.no_grad():
        y = out(T(g['x'], cuda))
    assert_exact(y, g['out'], 'accumulated output')


def test_wide_cuba_recurrent_takes_the_stepwise_walk(cuda, slayer):
    """More neurons than the one-launch kernel holds: the block still runs, and on a width both
    paths cover they give the same spikes."""
    torch.manual_seed(3)
    rec = slayer.block.cuba.Recurrent(dict(CUBA_P), 16, 1040, weight_scale=2).to(cuda)
    x = (torch.rand(2, 16, 12, device=cuda) < 0.3).float()
    with torch.no_grad():
        y = rec(x)
    assert y.shape == (2, 1040, 12)
    from lava_dl_b200.slayer.utils import recurrent
    small = slayer.block.cuba.Recurrent(dict(CUBA_P), 16, 24, weight_scale=2).to(cuda)
    twin = slayer.block.cuba.Recurrent(dict(CUBA_P), 16, 24, weight_scale=2).to(cuda)
    twin.load_state_dict(small.state_dict())
    z = small.input_synapse(x)
    mat = small.neuron.quantize_8bit(small.recurrent_synapse.weight.reshape(24, 24))
    with torch.no_grad():
        fast = recurrent.recurrent_walk(z, small.neuron, mat)
        slow = recurrent._StepwiseRecurrent.apply(z, twin.neuron, mat)
    assert_exact(fast, slow, 'one-launch kernel against the stepwise walk')


def test_graphed_replay_of_an_inference_call(cuda, slayer):
    """``utils.Graphed`` replays a neuron's (and a block chain's) forward as one CUDA graph:
    the same spikes as the eager call on every new input, refused for persistent state."""
    gen = torch.Generator().manual_seed(5)
    neuron = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03).to(cuda)
    x0 = torch.empty(4, 96, 64).normal_(0.3, 1.0, generator=gen).to(cuda)
    graphed = slayer.utils.Graphed(neuron, x0)
    for _ in range(3):
        x = torch.empty(4, 96, 64).normal_(0.3, 1.0, generator=gen).to(cuda)
        with torch.no_grad():
            want = neuron(x)
        assert_exact(graphed(x), want, 'graphed neuron forward')
    net = torch.nn.Sequential(slayer.block.cuba.Dense(dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03), 96, 40),
                              slayer.block.cuba.Dense(dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03), 40, 10)).to(cuda)
    s0 = (torch.rand(4, 96, 64, generator=gen) < 0.2).float().to(cuda)
    gnet = slayer.utils.Graphed(net, s0)
    s1 = (torch.rand(4, 96, 64, generator=gen) < 0.2).float().to(cuda)
    with torch.no_grad():
        want = net(s1)
    assert_exact(gnet(s1), want, 'graphed chain of blocks')
    with pytest.raises(RuntimeError):
        graphed(torch.zeros(4, 96, 32, device=cuda))
    keeper = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03, persistent_state=True).to(cuda)
    with pytest.raises(RuntimeError):
        slayer.utils.Graphed(keeper, x0)


def test_packed_result_expanded_on_the_host_in_stream_order(cuda, slayer):
    """A packed inference result copied to the host as bits and expanded there by the library,
    queued on the copy's stream: once the stream is through, the host tensor is what ``forward``
    returns (1/32 of the bytes crossed PCIe)."""
    gen = torch.Generator().manual_seed(11)
    neuron = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03).to(cuda)
    x = torch.empty(3, 200, 333).normal_(0.3, 1.0, generator=gen).to(cuda)
    with torch.no_grad():
        want = neuron(x).cpu()
        bits = neuron.forward_packed(x)
    side = torch.cuda.Stream(cuda)
    side.wait_stream(torch.cuda.current_stream(cuda))
    bits_host = torch.empty(bits.shape, dtype=torch.int32, pin_memory=True)
    out = torch.full(want.shape, -1.0).pin_memory()
    with torch.cuda.stream(side):
        bits_host.copy_(bits, non_blocking=True)
        got = slayer.utils.unpack_spikes(bits_host, x.shape[-1], out=out, stream=side)
    side.synchronize()
    assert got is out
    assert_exact(out, want.numpy(), 'host expansion of the packed spikes')
    assert_exact(slayer.utils.unpack_spikes(bits_host, x.shape[-1]), want.numpy(), 'synchronous host expansion')
