"""Forward + backward of llsa_l1 / llsa_l2 for operands that live in pinned HOST memory.

Every batch element is independent (sparse_attention_res_2.py:179: all grids are (..., B*H)),
so the (batch, head) slices are cut into chunks (whole batch elements, or groups of heads of one batch
element) and three streams run a software pipeline over them:

    copy-in stream : q, k, v, d_o of chunk c+1   host -> device
    compute stream : the operator and its backward on chunk c
    copy-out stream: o, dq, dk, dv of chunk c-1  device -> host

PCIe carries both directions at once, so a step costs about max(bytes in, bytes out) / link
bandwidth instead of the sum of both copies plus the compute.  Device staging buffers are
allocated once per pipeline object; nothing here touches the default stream.

With graphs=True the forward + backward of a chunk is captured once per staging slot as a CUDA graph
(static operands, static results) and replayed per chunk: the host then spends a graph launch instead of
some twenty kernel launches plus autograd bookkeeping per chunk, which is what lets the chunks be small
(a few heads) and the unoverlapped first copy-in and last copy-out short.
"""
import torch


def capture_fwd_bwd(call, q, k, v, do, stream=None):
    """One forward + backward of `call(q, k, v)` against the upstream gradient `do`, captured as a CUDA graph on static
    device tensors: returns (graph, (o, dq, dk, dv)); graph.replay() recomputes the four results in place from whatever
    q, k, v, do hold by then.  A step then costs the host one graph launch instead of some fifteen kernel launches, the
    operator dispatch and the autograd bookkeeping, which is what bounds small problems (a few (b,h) slices per GPU)."""
    dev = q.device
    stream = stream or torch.cuda.Stream(dev)
    ql, kl, vl = [t.detach().requires_grad_(True) for t in (q, k, v)]
    stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(stream):                       # warm-up outside the capture: lazy initialisation, kernel attributes
        for _ in range(2):
            ql.grad = kl.grad = vl.grad = None
            call(ql, kl, vl).backward(do)
    torch.cuda.synchronize(dev)
    ql.grad = kl.grad = vl.grad = None
    g = torch.cuda.CUDAGraph()
    # thread-local error mode: other threads of the process (a communicator's watchdog polling its events, for one) may keep
    # calling the CUDA API while this thread captures
    with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
        o = call(ql, kl, vl)
        o.backward(do)
    return g, (o.detach(), ql.grad, kl.grad, vl.grad)


class HostPipeline:
    def __init__(self, call, shape, dtype, device, chunk_batch=1, chunk_heads=None, depth=3, graphs=False):
        """call(q, k, v) -> o on device tensors; shape = (B, H, N, D) of the full host operands.
        A chunk is `chunk_batch` batch elements, or, with chunk_heads (and chunk_batch = 1), `chunk_heads` heads
        of one batch element: smaller chunks shorten the unoverlapped first copy-in and last copy-out."""
        B, H, N, D = shape
        if B % chunk_batch:
            raise ValueError("chunk_batch must divide the batch")
        if chunk_heads is not None and (chunk_batch != 1 or H % chunk_heads):
            raise ValueError("chunk_heads needs chunk_batch = 1 and must divide the head count")
        self.call, self.B, self.H, self.cb, self.ch, self.depth = call, B, H, chunk_batch, chunk_heads or H, depth
        self.dev = device
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        self.slots = [[torch.empty((chunk_batch, self.ch, N, D), dtype=dtype, device=device) for _ in range(4)] for _ in range(depth)]
        self.graphs = [self._capture(slot) for slot in self.slots] if graphs else None
        self._out_done = [None] * depth        # the copy-out of a slot's static results has finished

    def _capture(self, slot):
        """(graph, (o, dq, dk, dv)) of one slot: leaves that alias the staging buffers, results in the graph's own pool."""
        q, k, v = [t.detach().requires_grad_(True) for t in slot[:3]]
        for t in slot:
            t.zero_()
        torch.cuda.synchronize(self.dev)
        with torch.cuda.stream(self.s_comp):               # warm-up outside the capture: lazy initialisation, autotuned attributes
            for _ in range(2):
                q.grad = k.grad = v.grad = None
                self.call(q, k, v).backward(slot[3])
        torch.cuda.synchronize(self.dev)
        q.grad = k.grad = v.grad = None
        g = torch.cuda.CUDAGraph()
        # thread-local error mode: other threads of the process (a communicator's watchdog polling its events, for one) may keep
        # calling the CUDA API while this thread captures
        with torch.cuda.graph(g, stream=self.s_comp, capture_error_mode="thread_local"):
            o = self.call(q, k, v)
            o.backward(slot[3])
        return g, (o.detach(), q.grad, k.grad, v.grad)

    def _chunks(self):
        for b0 in range(0, self.B, self.cb):
            for h0 in range(0, self.H, self.ch):
                yield (slice(b0, b0 + self.cb), slice(h0, h0 + self.ch))

    def fwd_bwd(self, hq, hk, hv, hdo, ho, hdq, hdk, hdv):
        """Pinned host tensors in, pinned host tensors out.  The work is ordered after what the current
        stream holds at the call and the current stream is made to wait for it, so the results are valid
        once the current stream has been synchronised."""
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        chunks = list(self._chunks())
        n_chunks = len(chunks)
        ev_in = [torch.cuda.Event() for _ in range(n_chunks)]
        ev_comp = [torch.cuda.Event() for _ in range(n_chunks)]
        ev_free = [None] * self.depth          # slot's device inputs no longer needed (its backward has run)
        keep = []
        for c in range(n_chunks):
            sl = chunks[c]
            slot = self.slots[c % self.depth]
            with torch.cuda.stream(self.s_in):
                if ev_free[c % self.depth] is not None:
                    self.s_in.wait_event(ev_free[c % self.depth])
                for d_, h_ in zip(slot, (hq, hk, hv, hdo)):
                    d_.copy_(h_[sl], non_blocking=True)
                ev_in[c].record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ev_in[c])
                if self.graphs is not None:
                    if self._out_done[c % self.depth] is not None:     # the replay overwrites the slot's static results
                        self.s_comp.wait_event(self._out_done[c % self.depth])
                    graph, outs = self.graphs[c % self.depth]
                    graph.replay()
                else:
                    q, k, v = [d_.detach().requires_grad_(True) for d_ in slot[:3]]
                    o = self.call(q, k, v)
                    o.backward(slot[3])
                    outs = (o.detach(), q.grad, k.grad, v.grad)
                ev_comp[c].record(self.s_comp)
                ev_free[c % self.depth] = ev_comp[c]
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_comp[c])
                for h_, d_ in zip((ho, hdq, hdk, hdv), outs):
                    if self.graphs is None:
                        d_.record_stream(self.s_out)
                    h_[sl].copy_(d_, non_blocking=True)
                if self.graphs is not None:
                    self._out_done[c % self.depth] = torch.cuda.Event()
                    self._out_done[c % self.depth].record(self.s_out)
            keep.append(outs)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_comp)
        self._keep = keep                      # device results stay referenced until the next call
        return ho, hdq, hdk, hdv
