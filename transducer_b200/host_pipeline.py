"""Loss and gradients for batches that live in HOST memory.

When emissions arrive in (pinned) host buffers and the gradients have to go back to the
host -- a joiner on another device, a data-loading process, an embedding in a
C++/Go/Java trainer through the C ABI -- the step is bound by the PCIe link, not by the
kernels: at the reference's benchmark shape 2.7 GB go in and 2.7 GB come out for 2.7 ms
of compute.  The link is full duplex, so this module cuts the batch into chunks of a few
utterances (they are independent) and runs them through a ring of slots, each with its
own stream and device buffers: while chunk i computes, chunk i+1 is on its way in and
the gradients of chunk i-1 are on their way out.  The step then costs about the larger
of the two directions instead of their sum.

No counterpart in the reference (its wrapper takes device tensors only,
transducer/torch_binding.py:23-58).  Same arithmetic, same kernels, same results as
`TransducerLoss` on the whole batch: utterances do not interact.
"""
import torch

from . import _transducer


class _Slot(object):
    def __init__(self, device):
        self.stream = torch.cuda.Stream(device=device)
        self.shape = None

    def fit(self, n, T, U, V, device, forward_only=False, dtype=torch.float32):
        if self.shape == (n, T, U, V, forward_only, dtype):
            return
        f32 = dict(device=device, dtype=torch.float32)
        io = dict(device=device, dtype=dtype)   # emissions, predictions and their gradients
        i32 = dict(device=device, dtype=torch.int32)
        u8 = dict(device=device, dtype=torch.uint8)
        self.E = torch.empty((n, T, V), **io)
        self.P = torch.empty((n, U, V), **io)
        self.labels = torch.empty((n, max(U - 1, 0)), **i32)
        self.il = torch.empty((n,), **i32)
        self.ll = torch.empty((n,), **i32)
        self.deltas = torch.empty((n,), **f32)
        self.costs = torch.empty((n,), **f32)
        self.eg = None if forward_only else torch.empty((n, T, V), **io)
        self.pg = None if forward_only else torch.empty((n, U, V), **io)
        self.saved_bytes = _transducer.loss_saved_bytes(n, T, U, V)
        self.saved = torch.empty(max(self.saved_bytes, 1), **u8)
        self.fwd_bytes = _transducer.loss_forward_workspace_bytes(n, T, U, V)
        self.bwd_bytes = 0 if forward_only else _transducer.loss_backward_workspace_bytes(n, T, U, V)
        self.ws = torch.empty(max(self.fwd_bytes, self.bwd_bytes, 1), **u8)
        self.shape = (n, T, U, V, forward_only, dtype)


class HostLossPipeline(object):
    """RNN-T loss forward + backward from host buffers to host buffers.

    Arguments:
        blank (int): id of the blank label.
        chunk (int): utterances per chunk (the unit that is copied and computed at once).
        slots (int): chunks in flight; 3 keeps one copying in, one computing and one
            copying out.
        device: CUDA device (default: the current one).
        forward_only (bool): compute the costs only (no gradients; pass None for egrads and
            pgrads).
        valid_rows_only (bool): move only the frames t < input_lengths[b] of the emissions and
            of their gradient, and only the positions u <= label_lengths[b] of the predictions
            and of theirs, over the link (the kernels never read the padding, and its gradient
            is zero by definition); the padding of egrads / pgrads is zero-filled on the host
            while the device works, so the outputs are complete either way.  Saves the padded
            share of the traffic: 12 % at lengths of 1500..2000 in 2000 frames.

    Call with host tensors (pinned memory, or the copies will not overlap):
        emissions float32 [B,T,V], predictions float32 [B,U+1,V], labels int32 [B,U],
        input_lengths, label_lengths int32 [B]; outputs costs float32 [B], egrads [B,T,V],
        pgrads [B,U+1,V]; optional deltas float32 [B] (upstream gradient, default ones).
        emissions, predictions and both gradient buffers may all be bfloat16 instead (half the
        bytes over the link; see TransducerLoss for the shapes that takes).
    The call is asynchronous like any CUDA work: it returns a 1-element device tensor with
    the sum of the costs; the outputs are complete once the current stream (which is made
    to wait for the pipeline) has been synchronised.
    """

    def __init__(self, blank=0, chunk=8, slots=3, device=None, forward_only=False,
                 valid_rows_only=False):
        if not torch.cuda.is_available():
            raise RuntimeError("transducer_b200 runs on CUDA devices only")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.blank = int(blank)
        self.chunk = int(chunk)
        self.slots = [_Slot(self.device) for _ in range(int(slots))]
        self.loss_parts = None
        self.forward_only = bool(forward_only)
        self.valid_rows_only = bool(valid_rows_only)

    def __call__(self, emissions, predictions, labels, input_lengths, label_lengths,
                 costs, egrads, pgrads, deltas=None):
        outs = (("costs", costs),) if self.forward_only else \
            (("costs", costs), ("egrads", egrads), ("pgrads", pgrads))
        for name, t in (("emissions", emissions), ("predictions", predictions),
                        ("labels", labels), ("input_lengths", input_lengths),
                        ("label_lengths", label_lengths)) + outs:
            if t.device.type != "cpu":
                raise ValueError("%s must be a host tensor" % name)
            if not t.is_contiguous():
                raise ValueError("%s must be contiguous" % name)
        B, T, V = emissions.shape
        U = predictions.shape[1]
        if not self.forward_only and (egrads.shape != emissions.shape or
                                      pgrads.shape != predictions.shape):
            raise ValueError("gradient buffers must have the shapes of their inputs")
        dtype = emissions.dtype
        if dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("emissions must be torch.float32 or torch.bfloat16")
        for name, t in (("predictions", predictions),) + (() if self.forward_only else
                                                           (("egrads", egrads), ("pgrads", pgrads))):
            if t.dtype is not dtype:
                raise TypeError("%s must be %s like emissions" % (name, dtype))
        bf = dtype is torch.bfloat16
        loss_forward = _transducer.loss_forward_bf16 if bf else _transducer.loss_forward
        loss_backward = _transducer.loss_backward_bf16 if bf else _transducer.loss_backward
        dev = self.device
        n_chunks = (B + self.chunk - 1) // self.chunk
        if self.loss_parts is None or self.loss_parts.numel() != max(n_chunks, 1):
            self.loss_parts = torch.zeros((max(n_chunks, 1),), device=dev, dtype=torch.float32)
        sparse = self.valid_rows_only
        if sparse:
            t_len = [min(int(x), T) for x in input_lengths.tolist()]
            u_len = [min(int(x) + 1, U) for x in label_lengths.tolist()]
        caller = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(caller)
        with torch.cuda.device(dev):
            for i in range(n_chunks):
                lo, hi = i * self.chunk, min(B, (i + 1) * self.chunk)
                n = hi - lo
                slot = self.slots[i % len(self.slots)]
                slot.stream.wait_event(start)
                with torch.cuda.stream(slot.stream):
                    slot.fit(self.chunk, T, U, V, dev, self.forward_only, dtype)  # views of n <= chunk rows below
                    if sparse:
                        for k in range(n):
                            slot.E[k, :t_len[lo + k]].copy_(emissions[lo + k, :t_len[lo + k]],
                                                            non_blocking=True)
                            slot.P[k, :u_len[lo + k]].copy_(predictions[lo + k, :u_len[lo + k]],
                                                            non_blocking=True)
                    else:
                        slot.E[:n].copy_(emissions[lo:hi], non_blocking=True)
                        slot.P[:n].copy_(predictions[lo:hi], non_blocking=True)
                    slot.labels[:n].copy_(labels[lo:hi], non_blocking=True)
                    slot.il[:n].copy_(input_lengths[lo:hi], non_blocking=True)
                    slot.ll[:n].copy_(label_lengths[lo:hi], non_blocking=True)
                    if deltas is None:
                        slot.deltas.fill_(1.0)
                    else:
                        slot.deltas[:n].copy_(deltas[lo:hi], non_blocking=True)
                    _transducer.set_stream(slot.stream.cuda_stream)
                    loss_forward(
                        slot.E.data_ptr(), slot.P.data_ptr(), slot.labels.data_ptr(),
                        slot.il.data_ptr(), slot.ll.data_ptr(), slot.costs.data_ptr(),
                        self.loss_parts[i:].data_ptr(), slot.saved.data_ptr(), slot.saved_bytes,
                        n, T, U, V, self.blank, slot.ws.data_ptr(), slot.fwd_bytes)
                    costs[lo:hi].copy_(slot.costs[:n], non_blocking=True)
                    if not self.forward_only:
                        loss_backward(
                            slot.E.data_ptr(), slot.P.data_ptr(), slot.labels.data_ptr(),
                            slot.il.data_ptr(), slot.ll.data_ptr(), slot.saved.data_ptr(),
                            slot.saved_bytes, slot.deltas.data_ptr(), slot.eg.data_ptr(),
                            slot.pg.data_ptr(), n, T, U, V, self.blank, slot.ws.data_ptr(),
                            slot.bwd_bytes)
                        if sparse:
                            for k in range(n):
                                egrads[lo + k, :t_len[lo + k]].copy_(slot.eg[k, :t_len[lo + k]],
                                                                     non_blocking=True)
                                pgrads[lo + k, :u_len[lo + k]].copy_(slot.pg[k, :u_len[lo + k]],
                                                                     non_blocking=True)
                        else:
                            egrads[lo:hi].copy_(slot.eg[:n], non_blocking=True)
                            pgrads[lo:hi].copy_(slot.pg[:n], non_blocking=True)
            for slot in self.slots:
                done = torch.cuda.Event()
                done.record(slot.stream)
                caller.wait_event(done)
            _transducer.set_stream(caller.cuda_stream)
        if sparse and not self.forward_only:
            # the padding of the gradients, on the host, while the device works (the copies
            # above touch other rows of the same buffers)
            for bb in range(B):
                if t_len[bb] < T:
                    egrads[bb, t_len[bb]:].zero_()
                if u_len[bb] < U:
                    pgrads[bb, u_len[bb]:].zero_()
        return self.loss_parts.sum().reshape(1)
