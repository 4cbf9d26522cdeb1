"""Host logic of the multi-GPU path on CPU: two gloo ranks shard a batch, each
computes its shard's spikes and shared-parameter gradients (with the oracle
standing in for the kernels, which need a GPU), and one flattened all-reduce
must reproduce the single-process result."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lava_dl_b200 import _dist


def test_shard_bounds_cover_the_batch():
    for n in (0, 1, 7, 8, 64, 65):
        for world in (1, 2, 3, 8):
            cuts = [_dist.shard_bounds(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, x, g, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        xs = _dist.shard_batch(torch.from_numpy(x)).numpy()
        gs = _dist.shard_batch(torch.from_numpy(g)).numpy()
        r = O.cuba(xs, 1.25, 1024.0, 123.0, grad_spike=gs)
        cd = torch.nn.Parameter(torch.tensor([1024.0]))
        vd = torch.nn.Parameter(torch.tensor([123.0]))
        frozen = torch.nn.Parameter(torch.tensor([7.0]), requires_grad=False)
        cd.grad = torch.tensor(r['grad_current_decay'], dtype=torch.float32)
        if rank == 0:  # a rank without a gradient must still join the same collective
            vd.grad = torch.tensor(r['grad_voltage_decay'], dtype=torch.float32)
            local_v = 0.0
        else:
            local_v = float(r['grad_voltage_decay'][0])
            vd.grad = None
        n = _dist.allreduce_param_grads([cd, frozen, vd])
        assert n == 2 and frozen.grad is None
        np.savez(os.path.join(out_dir, f'rank{rank}.npz'), spike=r['spike'], cd=cd.grad.numpy(), vd=vd.grad.numpy(),
                 missing_v=np.float64(local_v))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_single_process(tmp_path):
    from oracle import oracle as O
    rng = np.random.default_rng(7)
    x = rng.normal(0.3, 1.0, size=(5, 6, 64)).astype(np.float32)  # 5 samples: ragged split 3 + 2
    g = rng.normal(size=x.shape).astype(np.float32)
    full = O.cuba(x, 1.25, 1024.0, 123.0, grad_spike=g)
    port = _free_port()
    mp.spawn(_worker, args=(2, port, x, g, str(tmp_path)), nprocs=2, join=True)
    r0 = np.load(tmp_path / 'rank0.npz')
    r1 = np.load(tmp_path / 'rank1.npz')
    assert np.array_equal(np.concatenate([r0['spike'], r1['spike']]), full['spike'])  # no forward communication
    assert np.allclose(r0['cd'], r1['cd']) and np.allclose(r0['cd'], full['grad_current_decay'], rtol=1e-5)
    # rank 1 withheld its voltage-decay gradient: the reduced value is rank 0's share only
    assert np.allclose(r0['vd'], r1['vd'])
    assert np.allclose(r0['vd'] + r1['missing_v'], full['grad_voltage_decay'], rtol=1e-5)


def test_allreduce_is_a_no_op_without_a_process_group():
    p = torch.nn.Parameter(torch.tensor([1.0, 2.0]))
    p.grad = torch.tensor([0.5, 0.25])
    assert _dist.allreduce_param_grads([p]) == 2
    assert p.grad.tolist() == [0.5, 0.25]


def _leaving_worker(rank, world, port, out_dir):
    """Rank 1 leaves between steps (no collective in flight); rank 0 must get an error from its next
    all-reduce within the group's timeout instead of waiting forever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    p = torch.nn.Parameter(torch.tensor([1.0]))
    p.grad = torch.tensor([float(rank + 1)])
    _dist.allreduce_param_grads([p])          # step 1: both ranks
    assert p.grad.item() == 3.0
    if rank == 1:
        os._exit(0)                           # the rank is gone before step 2 starts
    time.sleep(0.5)
    t0 = time.time()
    try:
        p.grad = torch.tensor([1.0])
        _dist.allreduce_param_grads([p])      # step 2: the peer never joins
        outcome = 'returned'
    except Exception as e:                    # gloo reports the closed connection or the timeout
        outcome = 'raised ' + type(e).__name__
    with open(os.path.join(out_dir, 'rank0.txt'), 'w') as f:
        f.write(f'{outcome} {time.time() - t0:.1f}')
    os._exit(0)


def test_a_rank_that_leaves_between_steps_ends_the_next_collective_with_an_error(tmp_path):
    port = _free_port()
    ctx = mp.get_context('spawn')
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=60)
        assert not pr.is_alive(), 'a rank hung'
    outcome, seconds = (tmp_path / 'rank0.txt').read_text().split(' ', 1)[0], (tmp_path / 'rank0.txt').read_text().rsplit(' ', 1)[1]
    assert outcome == 'raised', (tmp_path / 'rank0.txt').read_text()
    assert float(seconds) < 30
