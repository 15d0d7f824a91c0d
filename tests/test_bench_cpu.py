"""CPU: the host logic of bench.py - the operator list of a step, launch counting, the chain
bound and which convs the probe would send to the event-driven kernel - on small workloads built
with the oracle as the operator set (no GPU, no CUDA extension)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


@pytest.fixture(scope="module")
def oracle_ops():
    return bench.OracleOps(threads=2)


def test_step_of_the_small_mlp_lists_its_operators(oracle_ops):
    wl = bench.build_workload(1, oracle_ops, torch.device("cpu"), batch_override=2)
    ops = [op for op, _, _, _ in wl.op_list(False)]
    assert ops.count("conv") == len(wl.layers) and ops.count("corr") == len(wl.layers)
    assert "getSpikes" in ops and "spikeGrad" in ops and "shift" in ops
    fused = [op for op, _, _, _ in wl.op_list(True)]
    assert "getSpikesDelayed" in fused and "spikeGradShift" in fused and "shift" not in fused
    # nothing here is large enough to be probed: one launch per operator
    assert wl.launches_per_step(False) == len(ops) and wl.launches_per_step(True) == len(fused)
    assert wl.sparse_convs(True) == {}
    assert wl.chain_bound_ms(True, 6449.4, 1965.0) > 0
    outs = wl.step(oracle_ops)
    assert all(o is None or torch.is_tensor(o) or isinstance(o, (tuple, list)) for o in outs)


def test_cnn_chain_fuses_corr_with_the_surrogate_of_the_layer_below(oracle_ops):
    wl = bench.build_workload(3, oracle_ops, torch.device("cpu"), batch_override=1)
    n = len(wl.layers)
    plain = [op for op, _, _, _ in wl.op_list(False)]
    assert plain.count("conv") == n and plain.count("getSpikes") == n and plain.count("spikeGrad") == n
    assert plain.count("corr") == n - 1                      # the network input needs no gradient
    fused = wl.op_list(True)
    names = [op for op, _, _, _ in fused]
    assert names.count("convPacked") == 0 or names.count("conv") == 0
    assert names.count("corrSpikeGrad") == n - 1 and names.count("corr") == 0
    assert names.count("spikeGrad") == 1                      # only the output layer keeps its own
    # a fused launch covers the rows of the layer below: same element count as the corr it replaces
    plain_corr = sorted(el for op, _, el, _ in wl.op_list(False) if op == "corr")
    assert sorted(el for op, _, el, _ in fused if op == "corrSpikeGrad") == plain_corr


def test_probe_rule_and_bound_of_an_event_driven_conv():
    assert not bench.conv_is_probed((1 << 25) - 1, 300, 77)
    assert bench.conv_is_probed(1 << 25, 300, 77)
    assert not bench.conv_is_probed(1 << 26, 32, 77) and not bench.conv_is_probed(1 << 26, 5000, 77)
    assert not bench.conv_is_probed(1 << 26, 300, 2000)
    assert set(bench.SPARSE_DENSITY) == {"conv", "convPacked"}
    for op in bench.ALG_BYTES:
        assert bench.kernel_of(op, 300) and bench.kernel_of(op, 1450)
