"""Host-side logic of the API mirror that needs no GPU: parameter scaling and
quantisation, shape/geometry derivation, state bookkeeping, and the refusal to
run on CPU tensors (there is no fallback path)."""

import numpy as np
import pytest
import torch

import lava_dl_b200.slayer as slayer
from lava_dl_b200 import _ops


def test_cuba_parameters_follow_the_reference_scaling():
    n = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03)
    assert n.threshold == 1.25 and n.w_scale == 64 and n.s_scale == 4096 and n.p_scale == 4096
    assert n.threshold_eps == 0.01 / 4096
    assert float(n.current_decay) == 1024.0
    assert abs(float(n.voltage_decay) - 0.03 * 4096) < 1e-3
    assert n.device_params == {'type': 'CUBA', 'iDecay': 1024, 'vDecay': 123, 'vThMant': 80, 'refDelay': 1,
                               'gradedSpike': False}
    assert not n.current_decay.requires_grad
    assert [k for k, _ in n.named_buffers()] == ['current_state', 'voltage_state']
    assert 'current_state' not in n.state_dict()  # non-persistent buffers, as in the reference
    assert set(n.state_dict()) == {'current_decay', 'voltage_decay'}


def test_threshold_is_quantised_to_the_weight_scale():
    n = slayer.neuron.cuba.Neuron(threshold=1.2345, current_decay=0.5, voltage_decay=0.5)
    assert n.threshold == int(1.2345 * 64) / 64
    assert n.v_th_mant == int(n.threshold * 64)
    assert n.weight_exponent == 0


def test_alif_and_adrf_registrations():
    a = slayer.neuron.alif.Neuron(1.0, 0.5, 0.2, 0.05, 0.1, 0.1)
    assert a.threshold_step == 0.5
    assert float(a.threshold_state) == 1.0
    assert a.device_params['vThStep'] == 32 and a.device_params['type'] == 'ALIF'
    r = slayer.neuron.adrf.Neuron(0.5, 0.25, 10, 0.1, 0.1, 0.1)
    assert r.device_params['type'] == 'ADRF_PHASE'
    assert abs(float(r.period) - 10) < 0.05
    assert abs(float(r.decay) - 0.1) < 1e-3
    with pytest.raises(AssertionError):
        slayer.neuron.rf.Neuron(0.5, 3, 0.1)  # period below 4
    with pytest.raises(AssertionError):
        slayer.neuron.cuba.Neuron(1.0, [0.1, 0.2], 0.1)  # range needs shared_param=False


def test_per_channel_ranges():
    n = slayer.neuron.cuba.Neuron(1.0, 0.25, [0.02, 0.04], shared_param=False)
    assert (n.current_decay_min, n.current_decay_max) == (0.25 * 0.99, 0.25 * 1.01)
    assert (n.voltage_decay_min, n.voltage_decay_max) == (0.02, 0.04)


def test_quantize_is_round_with_straight_through_gradient():
    q = slayer.utils.quantize
    x = torch.tensor([0.5, 1.5, 2.49, -0.5, 204.8], requires_grad=True)
    y = q(x)
    assert y.tolist() == [0.0, 2.0, 2.0, -0.0, 205.0]  # round half to even, as torch.round
    y.sum().backward()
    assert x.grad.tolist() == [1.0] * 5
    assert q(torch.tensor([0.26]), step=0.25).item() == 0.25
    assert q(torch.tensor([0.49]), step=0.25, mode=slayer.utils.QUANTIZE_MODE.FLOOR).item() == 0.25


def test_right_shift_to_zero():
    f = slayer.utils.int_utils.right_shift_to_zero
    x = torch.tensor([4097, -4097, 4095, -4095, 0, -8192], dtype=torch.int64)
    assert f(x, 12).tolist() == [1, -1, 0, 0, 0, -2]
    with pytest.raises(Exception):
        f(torch.tensor([1.0]), 1)


def test_geometry_derivation():
    g = _ops.geom(torch.empty(4, 6, 5, 3, 50), 6)
    assert (g.rows, g.T, g.rows_per_batch, g.decay_block) == (4 * 6 * 5 * 3, 50, 90, 15)
    g = _ops.geom(torch.empty(7, 40))
    assert (g.rows, g.T) == (7, 40)
    g = _ops.geom(torch.empty(33))
    assert (g.rows, g.T) == (1, 33)
    with pytest.raises(ValueError):
        _ops.geom(torch.empty(4, 6, 50), 5)


def test_state_broadcast():
    x = torch.empty(2, 3, 10)
    assert _ops.row_state(torch.tensor([0.5]), x).tolist() == [0.5] * 6
    s = torch.arange(6.0).reshape(2, 3)
    assert _ops.row_state(s, x).tolist() == list(range(6))


def test_cpu_tensors_are_refused():
    x = torch.zeros(2, 3, 16)
    n = slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        n(x)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        slayer.utils.time.shift(x, 3)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        slayer.utils.filter.conv(x, torch.ones(4))
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        slayer.spike.Spike.apply(x, 1.0, 1.0, 1.0, False, 0, 1)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        slayer.neuron.dynamics.leaky_integrator.dynamics(x, torch.tensor([100.0]), torch.zeros(1), 4096)


def test_shape_checks_happen_before_any_kernel():
    n = slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03)
    with pytest.raises(AssertionError, match='at least 3 dimensions'):
        n(torch.zeros(4, 16))
    r = slayer.neuron.rf.Neuron(0.5, 10, 0.1)
    with pytest.raises(AssertionError, match='does not match'):
        r((torch.zeros(2, 3, 16), torch.zeros(2, 3, 8)))


def test_fir_module_default_response():
    f = slayer.utils.filter.FIR(time_constant=8, length=64)
    assert f.filter.shape == (64,)
    assert np.allclose(f.filter.numpy(), np.exp(-np.arange(64) / 8), rtol=1e-6)


def test_persistent_state_helpers():
    li = slayer.neuron.dynamics.leaky_integrator
    at = slayer.neuron.dynamics.adaptive_threshold
    st = torch.tensor([1.0, 2.0])
    sp = torch.tensor([0.0, 3.0])
    assert li.persistent_state(st, sp).tolist() == [1.0, 0.0]
    assert at.persistent_ref_state(st, sp, torch.tensor([0.5, 0.5])).tolist() == [1.0, 3.0]
    assert at.persistent_th_state(st, sp, 0.25).tolist() == [1.0, 2.25]


def test_sigma_delta_host_side():
    """Constructor arithmetic, refusals and shape checks of the sigma-delta family (no kernel runs)."""
    import lava_dl_b200.slayer as slayer
    relu = torch.nn.functional.relu
    n = slayer.neuron.sigma_delta.Neuron(threshold=0.1, activation=relu, scale=1 << 6)
    assert n.w_scale == 64 and n.s_scale == 4096
    assert abs(float(n.threshold) - 6 / 64) < 1e-7            # int(0.1 * 64) / 64
    assert n.delta.scale == 4096 and n.graded_spike is True
    assert n.device_params == {'type': 'SDNN', 'activation': 'relu', 'vThMant': 6}
    assert slayer.neuron.sigma_delta.neuron_params({'vThMant': 32}, scale=64) == {'threshold': 0.5}
    with pytest.raises(NotImplementedError):
        slayer.axon.Delta(threshold=0.5, cum_error=True)
    d = slayer.axon.Delta(threshold=1e-6, scale=64)
    d.clamp()
    assert float(d.threshold) == 1 / 64
    with pytest.raises(AssertionError):
        slayer.dendrite.Sigma()(torch.zeros(4, 8))            # needs [batch, ..., time]
    with pytest.raises(RuntimeError):
        slayer.dendrite.Sigma()(torch.zeros(2, 3, 8))         # CPU tensor: no fallback
    with pytest.raises(RuntimeError):
        n(torch.zeros(2, 3, 8))
    assert slayer.dendrite.Sigma().device_params == {'type': 'SDNN', 'sigma_output': True}


def test_delay_fusable_bound():
    import lava_dl_b200.slayer as slayer
    assert slayer.axon.Delay(max_delay=None).fusable_steps is None
    assert slayer.axon.Delay(max_delay=62).fusable_steps == 62
    assert slayer.axon.Delay(sampling_time=2, max_delay=100).fusable_steps == 50


def test_recurrent_block_host_side():
    """Construction mirrors block.cuba.Recurrent of the reference; there is no CPU path (a CPU tensor is
    refused whichever walk would take it), and every family has its recurrent and winner-takes-all blocks."""
    import lava_dl_b200.slayer as slayer
    p = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03)
    blk = slayer.block.cuba.Recurrent(p, 6, 8, weight_scale=2, delay=True)
    assert blk.neuron.persistent_state is True and 'persistent_state' not in p
    assert blk.recurrent_synapse.weight.shape[:2] == (8, 8) and blk.input_synapse.weight.shape[:2] == (8, 6)
    assert blk.input_synapse.pre_hook_fx == blk.neuron.quantize_8bit
    assert blk.delay is not None
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        blk(torch.zeros(2, 6, 5))
    alif = slayer.neuron.alif.Neuron(1.0, 0.1, 0.3, 0.1, 0.9, 0.9, persistent_state=True)
    with pytest.raises(RuntimeError, match='no CPU fallback'):   # the stepwise walk calls the same kernels
        slayer.utils.recurrent.custom_recurrent(torch.zeros(2, 8, 5), alif, blk.recurrent_synapse)
    for fam in ('cuba', 'alif', 'rf', 'adrf', 'rf_iz', 'adrf_iz'):
        mod = getattr(slayer.block, fam)
        assert set(mod.__all__) == {'Input', 'Flatten', 'Average', 'Dense', 'Conv', 'Pool', 'KWTA', 'Recurrent'}
    kw = slayer.block.cuba.KWTA(p, 6, 8, 3, self_excitation=1.7)
    kw.clamp()
    assert float(kw.self_excitation) == 1.0 and kw.neuron.persistent_state is True
    assert slayer.block.rf.Dense(dict(threshold=0.5, period=10, decay=0.1), 6, 4).synapse.complex is True
    avg = slayer.block.cuba.Average(2)
    assert torch.equal(avg(torch.arange(8.).reshape(1, 4, 2)), torch.tensor([[[1., 2.], [5., 6.]]]))


def test_replicate_matches_reference():
    """utils.time.replicate against the reference's interpolate-based version (values and gradient)."""
    import torch
    from _util import load_golden
    from lava_dl_b200.slayer.utils.time import replicate
    g = load_golden('replicate')
    for k, steps in (('2', 5), ('4', 3)):
        x = torch.tensor(g['x' + k], requires_grad=True)
        out = replicate(x, steps)
        assert out.shape == g['out' + k].shape
        assert (out.detach().numpy() == g['out' + k]).all()
        out.sum().backward()
        assert (x.grad == steps).all()
    with pytest.raises(NotImplementedError):
        replicate(torch.zeros(3), 4)


def test_unpack_spikes_on_the_host():
    """Packed spike words expanded on the CPU by the library (no GPU involved): every bit lands at
    step 32 w + i of its row, rows whose length is no multiple of 32 stop at T, any thread count."""
    import torch
    from lava_dl_b200 import _ops
    gen = torch.Generator().manual_seed(3)
    for shape, T in (((3, 5), 77), ((2, 4, 6), 64), ((7,), 1), ((1, 33), 300), ((0, 4), 40)):
        words = (T + 31) // 32
        bits = torch.randint(-2 ** 31, 2 ** 31 - 1, shape + (words,), generator=gen, dtype=torch.int64).to(torch.int32)
        shifts = torch.arange(32, dtype=torch.int32)
        want = ((bits.unsqueeze(-1) >> shifts) & 1).reshape(shape + (32 * words,))[..., :T].to(torch.float32)
        for threads in (1, 3, 0):
            got = _ops.unpack_spikes(bits, T, threads=threads)
            assert got.shape == want.shape and torch.equal(got, want)
        out = torch.full(shape + (T,), -1.0)
        assert _ops.unpack_spikes(bits, T, out=out) is out and torch.equal(out, want)
    with pytest.raises(ValueError):
        _ops.unpack_spikes(torch.zeros(2, 3, dtype=torch.int32), 200)
