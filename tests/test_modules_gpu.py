"""GPU: the Python operator modules (call conventions of the reference) and the mirror layer."""
import numpy as np
import pytest
import torch

import slayerpytorch_b200
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    return slayerpytorch_b200.load_ops()


def test_modules_are_the_native_build(ops):
    assert ops[0].backend == "slayer_b200" and ops[1].backend == "slayer_b200"
    assert ops[0].__file__.startswith(slayerpytorch_b200.lib_dir())


def test_shift_overloads_and_argument_conversion(ops):
    """Call patterns of the reference: (x, tensor, float) slayer.py:939; (x, -tensor, 0-dim cuda
    tensor) :957; (x, 4, 1) ints, test_slayer009.py:66-68; 1-element tensor -> scalar path."""
    sc = ops[0]
    x = torch.randn(2, 3, 2, 1, 50).cuda()
    xn = x.cpu().numpy()
    lut = (torch.rand(3, 2, 1) * 6 - 3).cuda()
    Ts0 = torch.tensor(0.5).cuda()
    np.testing.assert_array_equal(sc.shift(x, lut, 0.5).cpu().numpy(), co.shift(xn, lut.cpu().numpy(), 0.5))
    np.testing.assert_array_equal(sc.shift(x, -lut, Ts0).cpu().numpy(), co.shift(xn, -lut.cpu().numpy(), 0.5))
    np.testing.assert_array_equal(sc.shift(x, lut).cpu().numpy(), co.shift(xn, lut.cpu().numpy(), 1.0))
    np.testing.assert_array_equal(sc.shift(x, 4, 1).cpu().numpy(), co.shift(xn, 4, 1))
    np.testing.assert_array_equal(sc.shift(x, 2.0).cpu().numpy(), co.shift(xn, 2.0, 1))
    np.testing.assert_array_equal(sc.shift(x, torch.tensor([3.0]).cuda(), Ts0).cpu().numpy(), co.shift(xn, 3.0, 0.5))
    with pytest.raises(TypeError):
        sc.shift(x, "a")
    with pytest.raises(RuntimeError):
        sc.shift(x, lut.reshape(-1)[:4].contiguous(), 1.0)


def test_input_checks_raise_runtime_error(ops):
    sc, lc = ops
    x = torch.randn(1, 2, 1, 1, 16)
    f = torch.randn(3)
    with pytest.raises(RuntimeError):
        sc.conv(x, f.cuda(), 1.0)                       # CPU tensor
    with pytest.raises(RuntimeError):
        sc.conv(x.cuda()[..., ::2], f.cuda(), 1.0)         # not contiguous
    with pytest.raises(RuntimeError):
        sc.corr(x.cuda().double(), f.cuda(), 1.0)       # not float32
    with pytest.raises(RuntimeError):
        lc.getSpikes(x, 0, 80, 1, 1, 1)
    with pytest.raises(TypeError):
        lc.getSpikes(x.cuda(), 0, 80.5, 1, 1, 1)        # float where an unsigned is expected
    with pytest.raises(TypeError):
        lc.getSpikes(x.cuda(), 0, -80, 1, 1, 1)
    with pytest.raises(RuntimeError):
        lc.getSpikes(x.cuda(), 0, 80, 1, 1, 0)          # refDelay = 0 is rejected


def test_get_spikes_updates_membrane_potential_in_place(ops):
    u = (torch.randn(1, 4, 1, 1, 100) * 8).cuda()
    before = u.clone()
    nu = torch.tensor([0.0, -20.0, -14.0, -8.0]).cuda()
    s = ops[0].getSpikes(u, nu, 10, 1)                  # ints convert to float like the reference
    assert s.sum() > 0 and not torch.equal(u, before)
    sw, uw = co.srm_get_spikes(before.cpu().numpy(), nu.cpu().numpy(), 10.0, 1.0)
    np.testing.assert_array_equal(s.cpu().numpy(), sw)
    np.testing.assert_array_equal(u.cpu().numpy(), uw)


def test_conv_accepts_any_rank_and_filter_shape(ops):
    x = torch.randn(6, 40).cuda()
    f = torch.randn(2, 3).cuda()
    got = ops[0].conv(x, f, torch.tensor(0.5).cuda())
    np.testing.assert_allclose(got.cpu().numpy(), co.conv(x.cpu().numpy(), f.cpu().numpy().ravel(), 0.5), rtol=1e-5, atol=1e-6)


def test_ops_run_on_the_current_stream(ops):
    x = torch.randn(64, 128, 1, 1, 300).cuda()
    f = torch.randn(77).cuda()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        y = ops[0].conv(x, f, 1.0)
        z = ops[0].shift(y, 3.0, 1.0)
    st.synchronize()
    want = co.shift(co.conv(x.cpu().numpy(), f.cpu().numpy(), 1.0), 3.0, 1.0)
    np.testing.assert_allclose(z.cpu().numpy(), want, rtol=1e-5, atol=1e-5)


def test_mirror_layer_gradient_kat(golden_dir):
    """test/test_slayer003.py through this package's own layer API."""
    from slayerpytorch_b200 import layer as L
    srm = np.load(golden_dir + "/srm_kat.npz")
    dev = torch.device("cuda")
    neuron = {"type": "SRMALPHA", "theta": 10, "tauSr": 1.0, "tauRef": 1.0, "scaleRef": 2, "tauRho": 0.1, "scaleRho": 1}
    sim = {"Ts": 0.1, "tSample": 50}
    net = L.spikeLayer(neuron, sim, fullRefKernel=True).to(dev)
    fc1, fc2 = net.dense(250, 25).to(dev), net.dense(25, 1).to(dev)
    fc1.weight = torch.nn.Parameter(torch.from_numpy(srm["w1Initial"]).reshape(25, 250, 1, 1, 1).to(dev))
    fc2.weight = torch.nn.Parameter(torch.from_numpy(srm["w2Initial"]).reshape(1, 25, 1, 1, 1).to(dev))

    def events(idx, n):
        x = np.zeros((n, 500), np.float32)
        for nid, tid in idx:
            if tid < 500:
                x[nid, tid] = 10.0
        return torch.from_numpy(x).reshape(1, n, 1, 1, 500).to(dev)

    out = net.spike(net.psp(fc2(net.spike(net.psp(fc1(events(srm["spikeIn"], 250)))))))
    err = net.psp(out - events(srm["spikeOut"], 1))
    loss = 0.5 * torch.sum(err ** 2) * 0.1
    loss.backward()
    g1 = fc1.weight.grad.reshape(25, 250).cpu().numpy()
    g2 = fc2.weight.grad.reshape(1, 25).cpu().numpy()
    assert np.linalg.norm(srm["gradW2Initial"] - g2) / g2.size < 1e-4
    assert np.linalg.norm(srm["gradW1Initial"] - g1) / g1.size < 1e-4


def test_mirror_delay_gradient_matches_hand_formula():
    """test/test_slayer010.py:72-80: delay gradient = -sum(error * d(psp)/dt) * Ts."""
    from slayerpytorch_b200 import layer as L
    ops0 = slayerpytorch_b200.load_ops()[0]
    dev = torch.device("cuda")
    neuron = {"type": "SRMALPHA", "theta": 10, "tauSr": 1.0, "tauRef": 1.0, "scaleRef": 2, "tauRho": 1, "scaleRho": 1}
    sim = {"Ts": 0.1, "tSample": 50}
    Ts = 0.1
    net = L.spikeLayer(neuron, sim).to(dev)
    g = torch.Generator().manual_seed(10)
    spike_in = ((torch.rand(5, 25, 1, 1, 500, generator=g) > 0.8).float() / Ts).to(dev)
    delay = net.delay((25, 1, 1)).to(dev)
    psp_delayed = delay(net.psp(spike_in))
    upstream = torch.randn(5, 25, 1, 1, 500, generator=g).to(dev)
    psp_delayed.backward(upstream)
    diff = torch.tensor([1.0, -1.0], device=dev) / Ts
    dpsp = ops0.conv(psp_delayed.detach(), diff, 1)
    want = -torch.sum(upstream * dpsp, [0, -1], keepdim=True).reshape(25, 1, 1) * Ts
    assert torch.norm(want - delay.delay.grad).item() < 1e-4 * max(1.0, torch.norm(want).item())


@pytest.mark.gpu
def test_delay_grad_operator_shapes_and_errors():
    ops0 = slayerpytorch_b200.load_ops()[0]
    g = torch.randn(3, 4, 2, 1, 50, device="cuda")
    o = torch.randn(3, 4, 2, 1, 50, device="cuda")
    r = ops0.delayGrad(g, o, 1.0)
    assert r.shape == (4, 2, 1)
    diff = torch.tensor([-1.0, 1.0], device="cuda")
    want = torch.sum(g * ops0.conv(o, diff, 1), [0, -1])
    assert torch.allclose(r, want, rtol=1e-4, atol=1e-4)
    assert ops0.delayGrad(g[:0], o[:0], 1.0).eq(0).all() and ops0.delayGrad(g[:0], o[:0], 1.0).shape == (4, 2, 1)
    with pytest.raises(RuntimeError):
        ops0.delayGrad(g, o[:2], 1.0)
    with pytest.raises(RuntimeError):
        ops0.delayGrad(g.cpu(), o.cpu(), 1.0)


def _chain_layer():
    from slayerpytorch_b200 import layer as L
    neuron = {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2, "tauRho": 1, "scaleRho": 1}
    return L.spikeLayer(neuron, {"Ts": 1.0, "tSample": 300}).cuda()


@pytest.mark.parametrize("small_bytes", [0, 100 * 1024, 1 << 30])     # all chunked / mixed / all whole-batch
@pytest.mark.parametrize("capture", [False, True, "pipeline"])
@pytest.mark.parametrize("batch,chunks", [(16, 4), (7, 3), (3, 8), (5, 1)])
def test_host_pipeline_matches_single_call(batch, chunks, capture, small_bytes):
    """Chunked, overlapped streaming of a host batch gives the bits of one call on the whole batch."""
    from slayerpytorch_b200.hoststream import HostPipeline
    net = _chain_layer()
    g = torch.Generator().manual_seed(batch * 10 + chunks)
    x = ((torch.rand(batch, 40, 1, 1, 300, generator=g) < 0.3).float() * 3).pin_memory()
    up = torch.randn(batch, 40, 1, 1, 300, generator=g).pin_memory()
    delay = (torch.rand(40, generator=g) * 5).cuda()

    def step(xd, gd):
        xd = xd.detach().requires_grad_(True)
        y = net.delayShift(net.spike(net.psp(xd)), delay, 1.0)
        y.backward(gd)
        return y.detach(), xd.grad

    y_ref, gx_ref = step(x.cuda(), up.cuda())
    assert 0.005 < y_ref.mean().item() < 0.5
    y_h, gx_h = torch.empty_like(x).pin_memory(), torch.empty_like(x).pin_memory()
    pipe = HostPipeline("cuda", chunks=chunks, capture=capture, small_bytes=small_bytes)
    for _ in range(3):                     # later runs reuse the staging buffers (and graphs)
        y_h.fill_(-1)
        gx_h.fill_(-1)
        pipe.run(step, [x, up], [y_h, gx_h])
        torch.cuda.synchronize()
        assert torch.equal(y_h, y_ref.cpu())
        assert torch.equal(gx_h.view(torch.int32), gx_ref.cpu().view(torch.int32))


def test_host_pipeline_rejects_mismatched_batches():
    from slayerpytorch_b200.hoststream import HostPipeline
    pipe = HostPipeline("cuda", chunks=2)
    with pytest.raises(ValueError):
        pipe.run(lambda a, b: a, [torch.zeros(4, 3), torch.zeros(5, 3)], [torch.zeros(4, 3)])
    with pytest.raises(ValueError):
        pipe.run(lambda a: (a, a), [torch.zeros(4, 3).pin_memory()], [torch.zeros(4, 3).pin_memory()])
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        HostPipeline("cpu")


def test_operator_chain_replays_from_a_cuda_graph():
    """After one eager call per operator (set-up of per-device state), the chain captures into a
    CUDA graph and every replay reproduces the eager results."""
    ops0 = slayerpytorch_b200.load_ops()[0]
    from slayerpytorch_b200.layer import alpha_kernel
    g = torch.Generator(device="cuda").manual_seed(3)
    srm = torch.tensor(alpha_kernel(10.0, 1.0, 300), device="cuda", dtype=torch.float32)
    ref = torch.tensor(alpha_kernel(1.0, 1.0, 300, mult=-20.0), device="cuda", dtype=torch.float32)
    x = (torch.rand(8, 64, 1, 1, 300, device="cuda", generator=g) < 0.3).float() * 3
    up = torch.randn(8, 64, 1, 1, 300, device="cuda", generator=g)
    delay = torch.rand(64, device="cuda", generator=g) * 5

    def chain():
        u = ops0.conv(x, srm, 1.0)
        s = ops0.getSpikes(u, ref, 10.0, 1.0)
        d = ops0.shift(s, delay, 1.0)
        b = ops0.corr(ops0.spikeGrad(ops0.shift(up, -delay, 1.0), u, 10.0, 10.0, 1.0), srm, 1.0)
        return d, b, ops0.delayGrad(up, d, 1.0)

    want = [t.clone() for t in chain()]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = chain()
    for _ in range(3):
        for t in outs:
            t.fill_(7.0)
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(outs, want):
            assert torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("learnable", [True, False])
def test_spike_delayed_matches_the_two_separate_nodes(learnable):
    """spikeDelayed == delay(spike(u)) in outputs and in every gradient, bit for bit."""
    net = _chain_layer()
    g = torch.Generator().manual_seed(5)
    x = ((torch.rand(6, 40, 1, 1, 300, generator=g) < 0.3).float() * 3).cuda()
    up = torch.randn(6, 40, 1, 1, 300, generator=g).cuda()
    if learnable:
        dl_a, dl_b = net.delay(40).cuda(), net.delay(40).cuda()
        with torch.no_grad():
            dl_a.delay.copy_(torch.rand(40, 1, 1, generator=g) * 6)
            dl_b.delay.copy_(dl_a.delay)
    else:
        fixed = (torch.rand(40, generator=g) * 6).cuda()

    xa = x.clone().requires_grad_(True)
    ua = net.psp(xa)
    ya = dl_a(net.spike(ua)) if learnable else net.delayShift(net.spike(ua), fixed, 1.0)
    ya.backward(up)

    xb = x.clone().requires_grad_(True)
    ub = net.psp(xb)
    yb = net.spikeDelayed(ub, dl_b if learnable else fixed)
    yb.backward(up)

    assert 0.005 < ya.mean().item() < 0.5
    assert torch.equal(ya, yb)
    assert torch.equal(xa.grad.view(torch.int32), xb.grad.view(torch.int32))
    if learnable:
        assert torch.equal(dl_a.delay.grad, dl_b.delay.grad)


def test_num_spikes_loss_against_a_host_restatement():
    """numSpikes on the device vs the same formula written out with NumPy in float64
    (src/spikeLoss.py:84-104): count error inside the target region, psp of the spikes outside."""
    from slayerpytorch_b200 import loss as ours_loss
    from slayerpytorch_b200.layer import alpha_kernel
    Ts, T = 1.0, 300
    params = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
                         "tauRho": 1, "scaleRho": 1},
              "simulation": {"Ts": Ts, "tSample": T, "nSample": 12},
              "training": {"error": {"type": "NumSpikes", "tgtSpikeRegion": {"start": 40, "stop": 260},
                                     "tgtSpikeCount": {True: 60, False: 10}}}}
    g = torch.Generator().manual_seed(12)
    spikes = (torch.rand(5, 10, 1, 1, T, generator=g) < 0.1).float()
    label = torch.randint(0, 10, (5,), generator=g)
    desired = torch.zeros(5, 10, 1, 1, 1)
    desired[torch.arange(5), label] = 1
    err = ours_loss.spikeLoss(params).cuda()
    x = spikes.cuda().requires_grad_(True)
    loss = err.numSpikes(x, desired.cuda())
    loss.backward()

    s = spikes.numpy().astype(np.float64)
    inside = np.zeros(T)
    inside[40:260] = 1
    want_count = np.where(desired.numpy() == 1, 60.0, 10.0)
    count_err = (s[..., 40:260].sum(-1, keepdims=True) * Ts - want_count) / 220
    k = np.asarray(alpha_kernel(10.0, Ts, T), np.float64)
    outside = s * (1 - inside)
    psp = np.zeros_like(s)
    for i, kv in enumerate(k):
        psp[..., i:] += kv * outside[..., :T - i]
    e = psp * Ts + count_err * inside
    want = 0.5 * (e ** 2).sum() * Ts
    assert abs(loss.item() - want) <= 1e-5 * want
    # gradient = corr(error) everywhere (the part inside the region is a constant, not masked)
    grad = np.zeros_like(s)
    for i, kv in enumerate(k):
        grad[..., :T - i] += kv * e[..., i:]
    np.testing.assert_allclose(x.grad.cpu().numpy(), grad * Ts * Ts, rtol=2e-4, atol=1e-5)
    assert ours_loss.spikeClassifier.getClass(x.detach()).shape == (5,)


@pytest.mark.parametrize("Ts,region,shape", [(1.0, (0, 300), (64, 10, 1, 1, 300)), (1.0, (40, 260), (5, 10, 1, 1, 300)),
                                             (0.5, (10, 120), (3, 4, 2, 2, 300)), (1.0, (0, 2000), (2, 7, 1, 1, 2000))])
def test_num_spikes_loss_fused_kernel_equals_the_tensor_expressions(Ts, region, shape):
    """The one-kernel numSpikes (value and gradient) against the tensor-expression form of the
    same module, which follows src/spikeLoss.py:85-104 line by line: loss within 1e-6, gradient
    within 1e-5 of its largest entry; and a scaled upstream gradient scales the result."""
    from slayerpytorch_b200 import loss as ours_loss
    T = shape[-1]
    params = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
                         "tauRho": 1, "scaleRho": 1},
              "simulation": {"Ts": Ts, "tSample": int(T * Ts), "nSample": 12},
              "training": {"error": {"type": "NumSpikes", "tgtSpikeRegion": {"start": region[0], "stop": region[1]},
                                     "tgtSpikeCount": {True: 60, False: 10}}}}
    g = torch.Generator().manual_seed(T + shape[0])
    spikes = ((torch.rand(shape, generator=g) < 0.08).float() / Ts).cuda()
    desired = (torch.rand(shape[:2] + (1, 1, 1), generator=g) < 0.2).float()
    results = []
    for fused in (True, False):
        err = ours_loss.spikeLoss(params).cuda()
        err.fused = fused
        x = spikes.clone().requires_grad_(True)
        loss = err.numSpikes(x, desired, 0.7)
        (3.0 * loss).backward()
        results.append((loss.detach(), x.grad))
    (la, ga), (lb, gb) = results
    assert la.dtype == torch.float32 and la.dim() == 0
    torch.testing.assert_close(la, lb, rtol=1e-6, atol=0)
    torch.testing.assert_close(ga, gb, rtol=1e-5, atol=1e-5 * gb.abs().max().item())
    assert ga.abs().sum() > 0


def test_loihi_spike_delayed_layer_function_equals_the_two_steps():
    """layer.spikeLoihiDelayed = delayShift(spikeLoihi(w), 1): same forward bits, same gradient."""
    from slayerpytorch_b200 import layer as L
    neuron = {"type": "LOIHI", "vThMant": 80, "vDecay": 128, "iDecay": 1024, "refDelay": 1, "wgtExp": 0,
              "tauRho": 1, "scaleRho": 1}
    net = L.loihiLayer(dict(neuron), {"Ts": 1.0, "tSample": 1450}).cuda()
    g = torch.Generator().manual_seed(21)
    w = (torch.randint(-60, 60, (2, 6, 3, 3, 1450), generator=g) * (torch.rand(2, 6, 3, 3, 1450, generator=g) < 0.3)).float().cuda()
    gout = torch.randn(2, 6, 3, 3, 1450, generator=g).cuda()
    for steps in (1, 3):
        a = w.clone().requires_grad_(True)
        ya = net.delayShift(net.spikeLoihi(a), float(steps), 1.0)
        ya.backward(gout)
        b = w.clone().requires_grad_(True)
        yb = net.spikeLoihiDelayed(b, steps)
        yb.backward(gout)
        assert torch.equal(ya, yb) and ya.sum() > 0
        assert torch.equal(a.grad, b.grad)
