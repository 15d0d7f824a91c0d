"""CPU, gloo, world size 2: batch sharding + all-reduce(SUM) reproduce the single-process result.

The GPU kernels cannot run here, so each rank computes its shard with the CPU oracle; what is
under test is the host logic of slayerpytorch_b200.sharding (slice bounds, SUM reduction).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from slayerpytorch_b200 import sharding


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def chain(a, g, w, delay, srm, ref):
    """Hidden-layer hot path on the oracle; returns delayed spikes, input gradient, and a
    'weight gradient' (sum over batch and time) and the delay gradient."""
    from oracle import cpu_oracle as co
    u = co.conv(a, srm, 1.0)
    s, u = co.srm_get_spikes(u, ref, 10.0, 1.0)
    d = co.shift(s, delay, 1.0)
    gb = co.shift(g, -delay, 1.0)
    gi = co.corr(co.spike_grad(gb, u, 10.0, 10.0, 1.0), srm, 1.0)
    grad_w = np.einsum("nct,ndt->cd", gi[:, :, 0, 0, :], w[:, :, 0, 0, :]).astype(np.float32)
    diff = co.conv(d, np.array([-1.0, 1.0], np.float32), 1)
    grad_delay = np.sum(g * diff, axis=(0, -1)).reshape(-1).astype(np.float32)
    return d, gi, grad_w, grad_delay


def make_data():
    rng = np.random.RandomState(5)
    N, C, T = 6, 8, 64
    a = (np.abs(rng.randn(N, C, 1, 1, T)) * 2.5 * (rng.rand(N, C, 1, 1, T) < 0.4)).astype(np.float32)
    g = rng.randn(N, C, 1, 1, T).astype(np.float32)
    w = rng.randn(N, 5, 1, 1, T).astype(np.float32)
    delay = (rng.rand(C) * 4).astype(np.float32)
    srm = np.array([0, .5, .9, 1, .8, .5, .3, .1], np.float32)
    ref = np.array([-0.0, -20, -12, -6, -2], np.float32)
    return a, g, w, delay, srm, ref


def worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a, g, w, delay, srm, ref = make_data()
        ta, tg, tw = (sharding.shard_batch(torch.from_numpy(x)) for x in (a, g, w))
        d, gi, gw, gd = chain(ta.numpy(), tg.numpy(), tw.numpy(), delay, srm, ref)
        grads = [torch.from_numpy(gw), torch.from_numpy(gd)]
        sharding.allreduce_sum_(grads)
        lo, hi = sharding.shard_bounds(a.shape[0], rank, world)
        torch.save({"lo": lo, "hi": hi, "d": d, "gi": gi, "gw": grads[0].numpy(), "gd": grads[1].numpy()},
                   os.path.join(out, "rank%d.pt" % rank))
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_the_batch_exactly():
    for n in (1, 4, 7, 64, 65):
        for world in (1, 2, 3, 8):
            cuts = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.timeout(120)
def test_two_ranks_reproduce_single_process(tmp_path):
    world = 2
    mp.spawn(worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    a, g, w, delay, srm, ref = make_data()
    d, gi, gw, gd = chain(a, g, w, delay, srm, ref)
    parts = [torch.load(os.path.join(str(tmp_path), "rank%d.pt" % r), weights_only=False) for r in range(world)]
    for p in parts:
        np.testing.assert_array_equal(p["d"], d[p["lo"]:p["hi"]])        # spikes bit-identical per sample
        np.testing.assert_array_equal(p["gi"], gi[p["lo"]:p["hi"]])
        np.testing.assert_allclose(p["gw"], gw, rtol=1e-5, atol=1e-5)    # fp32 reduction order only
        np.testing.assert_allclose(p["gd"], gd, rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(parts[0]["gw"], parts[1]["gw"])
