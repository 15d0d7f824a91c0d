"""GPU, NCCL, one process per GPU: a batch-sharded training step equals the single-process step.

Each rank runs the SRM network 96-64-10 (psp, spike, learnable delay, spike-count loss) on its
contiguous share of the batch through ``slayerpytorch_b200.layer``; weight and delay gradients
are summed over the ranks with ``sharding.allreduce_sum_`` (SUM, because the reference's losses
and its delay gradient are sums over the batch: src/spikeLoss.py:58, :104, src/slayer.py:954).
Spikes must be bit-identical per sample and the reduced gradients must match the one-process
gradients to fp32 reduction-order tolerance.  Skipped with fewer than two visible GPUs; the host
logic is also covered on CPU ranks (gloo) in test_sharding_cpu.py.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

PARAMS = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
                     "tauRho": 1, "scaleRho": 1},
          "simulation": {"Ts": 1.0, "tSample": 300},
          "training": {"error": {"type": "NumSpikes", "tgtSpikeRegion": {"start": 0, "stop": 300},
                                 "tgtSpikeCount": {True: 60, False: 10}}}}
BATCH, N_IN, N_HID, N_OUT, T = 12, 96, 64, 10, 300


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_data():
    g = torch.Generator().manual_seed(2024)
    x = (torch.rand(BATCH, N_IN, 1, 1, T, generator=g) < 0.1).float()
    w1 = torch.randn(N_HID, N_IN, 1, 1, 1, generator=g) * 1.2
    w2 = torch.randn(N_OUT, N_HID, 1, 1, 1, generator=g) * 1.5
    delay = torch.rand(N_HID, 1, 1, generator=g) * 5
    label = torch.randint(0, N_OUT, (BATCH,), generator=g)
    desired = torch.zeros(BATCH, N_OUT, 1, 1, 1)
    desired[torch.arange(BATCH), label] = 1
    return x, w1, w2, delay, desired


def training_step(device, x, w1, w2, delay, desired):
    from slayerpytorch_b200 import layer as L
    from slayerpytorch_b200 import loss as loss_mod
    net = L.spikeLayer(dict(PARAMS["neuron"]), dict(PARAMS["simulation"])).to(device)
    fc1, fc2, dl = net.dense(N_IN, N_HID).to(device), net.dense(N_HID, N_OUT).to(device), net.delay(N_HID).to(device)
    with torch.no_grad():
        fc1.weight.copy_(w1)
        fc2.weight.copy_(w2)
        dl.delay.copy_(delay)
    hidden = net.spikeDelayed(net.psp(fc1(x.to(device))), dl)
    out = net.spike(net.psp(fc2(hidden)))
    loss = loss_mod.spikeLoss(PARAMS).to(device).numSpikes(out, desired.to(device))
    loss.backward()
    return hidden.detach(), out.detach(), loss.detach(), [fc1.weight.grad, fc2.weight.grad, dl.delay.grad]


def worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from slayerpytorch_b200 import sharding
        x, w1, w2, delay, desired = make_data()
        lo, hi = sharding.shard_bounds(BATCH, rank, world)
        hidden, out, loss, grads = training_step(device, sharding.shard_batch(x), w1, w2, delay,
                                                 sharding.shard_batch(desired))
        sharding.allreduce_sum_(grads + [loss])
        torch.cuda.synchronize()
        torch.save({"lo": lo, "hi": hi, "hidden": hidden.cpu(), "out": out.cpu(), "loss": loss.cpu(),
                    "grads": [g.cpu() for g in grads]}, "%s.%d" % (out_path, rank))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_training_step_equals_single_process(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d visible GPUs" % world)
    x, w1, w2, delay, desired = make_data()
    hidden, out, loss, grads = training_step(torch.device("cuda", 0), x, w1, w2, delay, desired)
    assert out.sum() > 0 and hidden.sum() > 0
    path = str(tmp_path / "rank")
    mp.spawn(worker, args=(world, free_port(), path), nprocs=world, join=True)
    parts = [torch.load("%s.%d" % (path, r)) for r in range(world)]
    for p in parts:                         # spikes of every sample: identical bits
        assert torch.equal(p["hidden"], hidden[p["lo"]:p["hi"]].cpu())
        assert torch.equal(p["out"], out[p["lo"]:p["hi"]].cpu())
    for p in parts:                         # every rank holds the same reduced values
        torch.testing.assert_close(p["loss"], loss.cpu(), rtol=1e-5, atol=0)
        for got, want in zip(p["grads"], grads):
            scale = want.abs().max().item()
            assert scale > 0
            torch.testing.assert_close(got, want.cpu(), rtol=1e-5, atol=1e-5 * scale)
        for got, first in zip(p["grads"], parts[0]["grads"]):
            assert torch.equal(got, first)
