"""Decode steps whose inputs live in pinned host memory.

The decode path itself takes device tensors (the serving engine hands it the projection output, which is already in HBM).
A caller that holds the step's inputs on the host -- a test harness, an offline replay of recorded activations, the
end-to-end leg of the benchmark -- would otherwise serialise, per step, three host->device copies, the two kernels and
one device->host copy on one stream.  HostStagedDecoder overlaps them: the copies of step t+1 run on their own stream
into the next of a few device buffers while step t computes, and the result of step t-1 drains on a third stream, so a
step costs max(copy in, compute, copy out) instead of their sum.  The host->device and device->host directions use
separate copy engines and the two directions of the PCIe link.

The arithmetic is LeapQuantState.decode, untouched; only the staging around it lives here.
"""
import torch


class HostStagedDecoder:
    """Double-buffered host staging around LeapQuantState.decode for one layer's state.

    submit() is asynchronous: it enqueues the copies and the kernels and returns.  drain() waits for everything that was
    submitted.  The host tensors must be pinned and must stay unchanged (inputs) / unread (output) until the matching
    slot is reused, i.e. until `depth` later submits have been drained or drain() has returned."""

    def __init__(self, state, ssm, A_log, dt_bias, idx, mixed_like, a_like, b_like, out_like, depth=4):
        dev = ssm.device
        if dev.type != "cuda":
            raise RuntimeError("HostStagedDecoder needs the state on a CUDA device")
        self.state, self.ssm, self.idx = state, ssm, idx
        self.A_log = A_log.to(device=dev, dtype=torch.float32)
        self.dt_bias = dt_bias.to(device=dev, dtype=torch.float32)
        self.depth = depth
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        mk = lambda like: [torch.empty(like.shape, dtype=like.dtype, device=dev) for _ in range(depth)]
        self.out = mk(out_like)
        # device input buffers: one slab per slot, laid out like host_slab(), with the three tensors as views into it
        sizes = [t.numel() * t.element_size() for t in (mixed_like, a_like, b_like)]
        o1 = (sizes[0] + 255) & ~255
        o2 = (o1 + sizes[1] + 255) & ~255
        total = (o2 + sizes[2] + 255) & ~255
        self.dslab = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(depth)]
        cut = lambda sl, o, n, t: sl[o:o + n].view(t.dtype).view(t.shape)
        self.mixed = [cut(sl, 0, sizes[0], mixed_like) for sl in self.dslab]
        self.a = [cut(sl, o1, sizes[1], a_like) for sl in self.dslab]
        self.b = [cut(sl, o2, sizes[2], b_like) for sl in self.dslab]
        ev = lambda: [torch.cuda.Event() for _ in range(depth)]
        self.ev_in, self.ev_done, self.ev_out = ev(), ev(), ev()
        self.n = 0

    @staticmethod
    def host_slab(mixed_like, a_like, b_like, steps=1):
        """Pinned host memory for `steps` decode steps whose three inputs lie back to back, and the views (mixed, a, b) of
        each step: submit() then moves a step's inputs with ONE host->device copy instead of three."""
        sizes = [t.numel() * t.element_size() for t in (mixed_like, a_like, b_like)]
        offs = [0, (sizes[0] + 255) & ~255]
        offs.append((offs[1] + sizes[1] + 255) & ~255)
        total = (offs[2] + sizes[2] + 255) & ~255
        slab = torch.empty(steps, total, dtype=torch.uint8).pin_memory()
        views = []
        for i in range(steps):
            views.append(tuple(slab[i, o:o + n].view(t.dtype).view(t.shape) for o, n, t in zip(offs, sizes, (mixed_like, a_like, b_like))))
        return slab, views

    def _slab_of(self, h_mixed, h_a, h_b):
        """The byte range that holds the three host tensors back to back (as laid out by host_slab), or None."""
        p0 = h_mixed.data_ptr()
        sizes = [t.numel() * t.element_size() for t in (h_mixed, h_a, h_b)]
        o1 = (sizes[0] + 255) & ~255
        o2 = (o1 + sizes[1] + 255) & ~255
        if h_a.data_ptr() - p0 == o1 and h_b.data_ptr() - p0 == o2:
            return o1, o2, o2 + sizes[2]
        return None

    def submit(self, h_mixed, h_a, h_b, h_out):
        """Enqueue one decode step: inputs from pinned host tensors, output into the pinned host tensor h_out."""
        s = self.n % self.depth
        reuse = self.n >= self.depth
        comp = torch.cuda.current_stream(self.ssm.device)
        with torch.cuda.stream(self.s_in):
            if reuse:
                self.s_in.wait_event(self.ev_done[s])            # the step that last read these input buffers is done
            lay = self._slab_of(h_mixed, h_a, h_b) if self.dslab is not None else None
            if lay is not None:                                  # inputs back to back on the host: one copy
                nbytes = lay[2]
                src = torch.as_strided(h_mixed.view(torch.uint8).view(-1), (nbytes,), (1,))
                self.dslab[s][:nbytes].copy_(src, non_blocking=True)
            else:
                self.mixed[s].copy_(h_mixed, non_blocking=True)
                self.a[s].copy_(h_a, non_blocking=True)
                self.b[s].copy_(h_b, non_blocking=True)
            self.ev_in[s].record(self.s_in)
        comp.wait_event(self.ev_in[s])
        if reuse:
            comp.wait_event(self.ev_out[s])                      # the previous result in this output buffer has drained
        self.state.decode(self.ssm, self.mixed[s], self.a[s], self.b[s], self.A_log, self.dt_bias, self.idx, self.out[s])
        self.ev_done[s].record(comp)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_done[s])
            h_out.copy_(self.out[s], non_blocking=True)
            self.ev_out[s].record(self.s_out)
        self.n += 1

    def drain(self):
        """Make the current stream wait for every submitted copy, then block the host until all of it has finished."""
        comp = torch.cuda.current_stream(self.ssm.device)
        for s in range(min(self.n, self.depth)):
            comp.wait_event(self.ev_out[s])
        comp.synchronize()

    def join(self):
        """Like drain() without blocking the host: the current stream waits for all outstanding output copies."""
        comp = torch.cuda.current_stream(self.ssm.device)
        for s in range(min(self.n, self.depth)):
            comp.wait_event(self.ev_out[s])
