"""Streaming a host-resident batch through the device operators.

The operators of this package work on device tensors.  A caller whose spike trains live in
host memory pays two PCIe transfers around every step, and on a B200 those transfers, not the
kernels, set the pace.  Rows of the ``[batch, ..., T]`` tensors are independent, so the batch
can be cut into chunks and the three phases of consecutive chunks overlapped::

    copy stream   : H2D(0) H2D(1) H2D(2) ...
    compute stream:        step(0) step(1) step(2) ...
    return stream :               D2H(0)  D2H(1)  D2H(2) ...

``HostPipeline`` does exactly that with three CUDA streams, three sets of device staging buffers
and events between the phases; there is no host-side synchronisation inside ``run``.  Results
are the same as those of one call on the whole batch, because every operator treats rows
independently (per-neuron tables are indexed inside a sample, and chunks hold whole samples).

Every copy over PCIe costs some tens of microseconds of set-up whatever its size, so tensors
whose chunks are small (below ``small_bytes`` per chunk, e.g. the ten output neurons of a
classifier next to its hidden layers) do not travel chunk by chunk: a small input crosses once
for the whole batch before the first chunk and is sliced on the device, a small output is
gathered on the device and crosses once after the last chunk.

A chunk's step is a handful of short kernels, so issuing them call by call can cost the host
more time than the copies take.  With ``capture=True`` the step is captured once per staging
slot into a CUDA graph (forward and backward alike) and every full-size chunk is one graph
launch; this requires a step without side effects other than its return values, because it is
run once on zero-filled buffers before capture.  ``capture="pipeline"`` goes one step further
and captures the whole of ``run`` - every chunk's copies, kernels and the events between the
three streams - into one graph per set of host buffers, so that a later ``run`` with the same
buffers is a single graph launch and the host's issue rate stops limiting the number of
chunks; the host tensors must then stay where they are (pinned, same addresses).  On a B200
with the benchmark's step the per-slot graphs are the faster of the two (2.1 ms against 2.3 ms
per step at 8 chunks): copies issued as graph nodes start a little later than copies issued on
a stream, which matters more than the host time saved.
"""
import torch


def chunk_bounds(batch, chunks):
    """``chunks`` nearly equal [start, stop) ranges covering ``range(batch)``; fewer when the
    batch is smaller than the number of chunks.  Sizes differ by at most one sample."""
    if batch < 0 or chunks < 1:
        raise ValueError("batch must be >= 0 and chunks >= 1")
    chunks = max(1, min(chunks, batch))
    base, extra = divmod(batch, chunks)
    bounds, start = [], 0
    for i in range(chunks):
        stop = start + base + (1 if i < extra else 0)
        bounds.append((start, stop))
        start = stop
    return bounds


class HostPipeline:
    """Overlaps host-to-device copies, a device step and device-to-host copies over chunks of
    the batch axis (axis 0).

    ``step`` is any callable taking the device chunks of the inputs (same order as
    ``host_inputs``) and returning a tensor or a tuple of tensors whose axis 0 is the chunk's
    batch; output k of every chunk is written to ``host_outputs[k][start:stop]``.  Host tensors
    should be pinned: copies from pageable memory are staged by the driver and do not overlap.
    """

    def __init__(self, device, chunks=8, capture=False, slots=3, small_bytes=256 * 1024):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("HostPipeline needs a CUDA device: the operators have no CPU path")
        self.chunks = int(chunks)
        self.copy_stream = torch.cuda.Stream(self.device)
        self.compute_stream = torch.cuda.Stream(self.device)
        self.return_stream = torch.cuda.Stream(self.device)
        self.capture = capture if capture == "pipeline" else bool(capture)
        self.slots = max(2, int(slots))      # sets of device staging buffers (and captured graphs)
        self.small_bytes = int(small_bytes)
        self._whole = {}                      # device copies of whole small tensors, by (role, index, shape)
        self._slots = None
        self._slot_key = None
        self._graphs = None            # per slot: (graph, static outputs), for the step in _graph_step
        self._graph_step = None
        self._pipeline_graphs = {}     # whole-run graphs by (step, host buffer addresses and shapes)

    def _staging(self, host_inputs, rows):
        key = tuple((tuple(t.shape[1:]), t.dtype) for t in host_inputs) + (rows,)
        if self._slot_key != key:
            self._slots = [[torch.empty((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.device)
                            for t in host_inputs] for _ in range(self.slots)]
            self._slot_key = key
            self._graphs = None
        return self._slots

    def _captured(self, step, slots):
        """One CUDA graph of ``step`` per staging slot, built on first use."""
        if self._graphs is not None and self._graph_step is step:
            return self._graphs
        graphs = []
        for bufs in slots:
            with torch.cuda.stream(self.compute_stream):
                for b in bufs:
                    b.zero_()
                step(*bufs)                                   # set-up calls happen outside the capture
            self.compute_stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.compute_stream):
                outs = step(*bufs)
            graphs.append((g, (outs,) if torch.is_tensor(outs) else tuple(outs)))
        self._graphs, self._graph_step = graphs, step
        return graphs

    def run(self, step, host_inputs, host_outputs):
        host_inputs, host_outputs = list(host_inputs), list(host_outputs)
        batch = host_inputs[0].shape[0]
        for t in host_inputs + host_outputs:
            if t.shape[0] != batch:
                raise ValueError("every host tensor must have the same batch size on axis 0")
        if batch == 0:
            return
        if self.capture != "pipeline":
            self._run(step, host_inputs, host_outputs, per_slot_graphs=bool(self.capture), keep=None)
            return
        key = (id(step),) + tuple((t.data_ptr(), tuple(t.shape), t.dtype) for t in host_inputs + host_outputs)
        entry = self._pipeline_graphs.get(key)
        if entry is None:
            for t in host_inputs + host_outputs:
                if not t.is_pinned():
                    raise ValueError("capture='pipeline' needs pinned host tensors")
            # once without capture: creates the staging buffers and any per-device state of the operators
            self._run(step, host_inputs, host_outputs, per_slot_graphs=False, keep=None)
            torch.cuda.current_stream(self.device).synchronize()
            keep = []                      # everything the captured work refers to stays alive with the graph
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._run(step, host_inputs, host_outputs, per_slot_graphs=False, keep=keep)
            entry = (graph, keep, step, host_inputs, host_outputs)
            self._pipeline_graphs[key] = entry
        entry[0].replay()

    def _run(self, step, host_inputs, host_outputs, per_slot_graphs, keep):
        batch = host_inputs[0].shape[0]
        bounds = chunk_bounds(batch, self.chunks)
        rows = max(b - a for a, b in bounds)
        caller = torch.cuda.current_stream(self.device)
        slots = self._staging(host_inputs, rows)
        graphs = self._captured(step, slots) if per_slot_graphs else None

        def chunk_bytes(t):
            return rows * (t.numel() // batch) * t.element_size()

        def whole(role, idx, t):           # persistent device buffer for a whole small tensor
            key = (role, idx, tuple(t.shape), t.dtype)
            if key not in self._whole:
                self._whole[key] = torch.empty(t.shape, dtype=t.dtype, device=self.device)
            return self._whole[key]

        many = len(bounds) > 1
        small_in = [many and chunk_bytes(t) < self.small_bytes for t in host_inputs]
        small_out = [many and chunk_bytes(t) < self.small_bytes for t in host_outputs]
        whole_in = [whole("in", i, t) if sm else None for i, (t, sm) in enumerate(zip(host_inputs, small_in))]
        whole_out = [whole("out", i, t) if sm else None for i, (t, sm) in enumerate(zip(host_outputs, small_out))]

        start = torch.cuda.Event()
        start.record(caller)
        for s in (self.copy_stream, self.compute_stream, self.return_stream):
            s.wait_event(start)
        small_ready = None
        if any(small_in):
            with torch.cuda.stream(self.copy_stream):
                for w, h in zip(whole_in, host_inputs):
                    if w is not None:
                        w.copy_(h, non_blocking=True)
                small_ready = torch.cuda.Event()
                small_ready.record(self.copy_stream)
            self.compute_stream.wait_event(small_ready)
        returned = [None] * self.slots     # recorded on the return stream when a slot's outputs are copied
        slot_free = [None] * self.slots    # recorded on the compute stream when a slot's step is enqueued
        for i, (a, b) in enumerate(bounds):
            k = i % self.slots
            dev_in = [buf[:b - a] for buf in slots[k]]
            with torch.cuda.stream(self.copy_stream):
                if slot_free[k] is not None:
                    self.copy_stream.wait_event(slot_free[k])
                for buf, h, sm in zip(dev_in, host_inputs, small_in):
                    if not sm:
                        buf.copy_(h[a:b], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.copy_stream)
            with torch.cuda.stream(self.compute_stream):
                self.compute_stream.wait_event(ready)
                for buf, w in zip(dev_in, whole_in):
                    if w is not None:
                        buf.copy_(w[a:b], non_blocking=True)          # device to device
                replay = graphs is not None and b - a == rows
                if replay:
                    if returned[k] is not None:              # the graph writes the same output buffers again
                        self.compute_stream.wait_event(returned[k])
                    graphs[k][0].replay()
                    outs = graphs[k][1]
                else:
                    outs = step(*dev_in)
                    if torch.is_tensor(outs):
                        outs = (outs,)
                if len(outs) != len(host_outputs):
                    raise ValueError("step returned %d tensors for %d host outputs" % (len(outs), len(host_outputs)))
                for o, w in zip(outs, whole_out):
                    if w is not None:
                        w[a:b].copy_(o[:b - a], non_blocking=True)    # gathered on the device
                done = torch.cuda.Event()
                done.record(self.compute_stream)
                slot_free[k] = done
            with torch.cuda.stream(self.return_stream):
                self.return_stream.wait_event(done)
                for o, h, sm in zip(outs, host_outputs, small_out):
                    if sm:
                        continue
                    if keep is not None:
                        keep.append(o)                       # captured: alive as long as the graph
                    elif not replay:
                        o.record_stream(self.return_stream)  # keeps the allocator from reusing it early
                    h[a:b].copy_(o[:b - a], non_blocking=True)
                if replay:
                    returned[k] = torch.cuda.Event()
                    returned[k].record(self.return_stream)
        with torch.cuda.stream(self.return_stream):         # `done` of the last chunk has been waited for
            for w, h in zip(whole_out, host_outputs):
                if w is not None:
                    h.copy_(w, non_blocking=True)
        finished = torch.cuda.Event()
        finished.record(self.return_stream)
        caller.wait_event(finished)
        tail = torch.cuda.Event()
        tail.record(self.compute_stream)
        caller.wait_event(tail)
        tail_copy = torch.cuda.Event()
        tail_copy.record(self.copy_stream)
        caller.wait_event(tail_copy)
