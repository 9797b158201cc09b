"""PyTorch surface of the library: the same names, arguments, checks and error
messages as awni/transducer's transducer/torch_binding.py, with every piece of
arithmetic (log-normalisers, lattice sweeps, gradient contractions) done by the
sm_100a kernels behind the `_transducer` module instead of torch ops.

CUDA tensors only: there is no CPU backend and no PyTorch fallback."""
import torch

from . import _transducer
from .errors import DeviceStatusError, raise_for_status  # noqa: F401


def check_device_status(device=None):
    """Synchronise torch's current stream on `device` and raise DeviceStatusError if a kernel
    of this library gave up on one of its bounded waits there since the last check (its
    outputs are then NaN / -1).  No counterpart in the reference, whose kernels never wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None \
        else torch.device(device)
    with DeviceManager(device):
        rc = _transducer.check_status()
        raise_for_status(rc, _transducer.last_error() if rc else "")


class DeviceManager(object):
    """Makes the tensors' device current for the duration of a native call
    (transducer/torch_binding.py:7-20) and points the library at torch's current
    stream on that device (the reference always used the legacy default stream)."""

    def __init__(self, device):
        if device.type != "cuda":
            raise ValueError("transducer_b200 runs on CUDA tensors only (got %s)" % device)
        self.device = device

    def __enter__(self):
        self.old_device = torch.cuda.current_device()
        torch.cuda.set_device(self.device)
        _transducer.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    def __exit__(self, exc_type, exc_value, traceback):
        torch.cuda.set_device(self.old_device)


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


class Transducer(torch.autograd.Function):
    """Autograd node for the loss (transducer/torch_binding.py:23-90)."""

    @staticmethod
    def forward(ctx, emissions, predictions, labels, input_lengths, label_lengths, blank=0,
                validate_lengths=True, check_status=False):
        certify_inputs(emissions, predictions, labels, input_lengths, label_lengths,
                       validate_lengths, allow_bf16=True)
        device = emissions.device
        emissions = emissions.contiguous()
        predictions = predictions.contiguous()
        B, T, V = emissions.shape
        U = predictions.shape[1]
        f32 = dict(device=device, dtype=torch.float32)
        costs = torch.empty((B,), **f32)
        loss_sum = torch.empty((1,), **f32)
        with DeviceManager(device):
            saved_bytes = _transducer.loss_saved_bytes(B, T, U, V)
            saved = _workspace(saved_bytes, device)
            nbytes = _transducer.loss_forward_workspace_bytes(B, T, U, V)
            ws = _workspace(nbytes, device)
            fwd = _transducer.loss_forward_bf16 if emissions.dtype is torch.bfloat16 \
                else _transducer.loss_forward
            fwd(
                emissions.data_ptr(), predictions.data_ptr(), labels.data_ptr(),
                input_lengths.data_ptr(), label_lengths.data_ptr(), costs.data_ptr(),
                loss_sum.data_ptr(), saved.data_ptr(), saved_bytes, B, T, U, V, blank,
                ws.data_ptr(), nbytes)
            if check_status:
                rc = _transducer.check_status()
                raise_for_status(rc, _transducer.last_error() if rc else "")
        # `saved` replaces the reference's saved alphas/log_norms/expEs/expPs/expLNs
        # (torch_binding.py:52-55); exp(emissions) is recomputed, never stored
        ctx.save_for_backward(emissions, predictions, saved, labels, input_lengths,
                              label_lengths)
        ctx.blank = blank
        ctx.check_status = check_status
        ctx.mark_non_differentiable(loss_sum)
        return costs, loss_sum

    @staticmethod
    def backward(ctx, deltas, _unused=None):
        emissions, predictions, saved, labels, input_lengths, label_lengths = ctx.saved_tensors
        device = emissions.device
        B, T, V = emissions.shape
        U = predictions.shape[1]
        deltas = deltas.to(torch.float32).contiguous()
        egrads = torch.empty((B, T, V), device=device, dtype=emissions.dtype)
        pgrads = torch.empty((B, U, V), device=device, dtype=emissions.dtype)
        with DeviceManager(device):
            nbytes = _transducer.loss_backward_workspace_bytes(B, T, U, V)
            ws = _workspace(nbytes, device)
            bwd = _transducer.loss_backward_bf16 if emissions.dtype is torch.bfloat16 \
                else _transducer.loss_backward
            bwd(
                emissions.data_ptr(), predictions.data_ptr(), labels.data_ptr(),
                input_lengths.data_ptr(), label_lengths.data_ptr(), saved.data_ptr(),
                saved.numel(), deltas.data_ptr(), egrads.data_ptr(), pgrads.data_ptr(),
                B, T, U, V, ctx.blank, ws.data_ptr(), nbytes)
            if ctx.check_status:
                rc = _transducer.check_status()
                raise_for_status(rc, _transducer.last_error() if rc else "")
        return egrads, pgrads, None, None, None, None, None, None


class TransducerLoss(torch.nn.Module):
    """The RNN-T loss for an additive joiner: the distribution at lattice node (t, u)
    is log_softmax(emissions[b, t, :] + predictions[b, u, :]).

    Same constructor and call signature as the reference's TransducerLoss
    (transducer/torch_binding.py:93-128).

    Arguments:
        blank (int, optional): id of the blank label (default 0).
        validate_lengths (bool, optional): compare the largest input / label length with the
            padded shapes, as the reference does (default).  That check reads two numbers back
            from the device, i.e. it synchronises the host with the stream on every call;
            pass False to skip it when the lengths are known to fit -- the call then only
            enqueues work (and can be captured in a CUDA graph).  No counterpart in the
            reference.
        check_status (bool, optional): after the forward and the backward kernels, wait for
            them and raise DeviceStatusError if one of them gave up on a bounded wait (see
            check_device_status).  Default: the value of validate_lengths -- the reference-style
            call synchronises once per call anyway; the enqueue-only call never does.
        reduction (str, optional): "none" (default; the reference returns the per-utterance
            costs, transducer/torch_binding.py:108-128), "sum" or "mean" over the batch.

    After each call ``last_loss_sum`` holds a detached 1-element device tensor with
    sum_b costs[b], produced by the kernel itself; a data-parallel caller can
    all-reduce it without launching a reduction.
    """

    def __init__(self, blank=0, validate_lengths=True, check_status=None, reduction="none"):
        super(TransducerLoss, self).__init__()
        if reduction not in ("none", "sum", "mean"):
            raise ValueError("reduction must be 'none', 'sum' or 'mean'")
        self.blank = blank
        self.validate_lengths = validate_lengths
        self.check_status = validate_lengths if check_status is None else bool(check_status)
        self.reduction = reduction
        self.last_loss_sum = None

    def forward(self, emissions, predictions, labels, input_lengths, label_lengths):
        """
        emissions    float32 [B, T, V]    unnormalised scores per frame
        predictions  float32 [B, U+1, V]  unnormalised scores per label position
                     (both may be bfloat16 instead: the loss is then computed in fp32 on the
                     exactly up-converted values and the gradients come back in bfloat16;
                     needs V % 8 == 0 and U + 1 <= 128)
        labels       int32   [B, U]       padded to the longest label sequence
        input_lengths, label_lengths  int32 [B]
        Returns costs float32 [B] (no reduction), differentiable w.r.t. emissions and
        predictions.
        """
        costs, loss_sum = Transducer.apply(
            emissions, predictions, labels, input_lengths, label_lengths, self.blank,
            self.validate_lengths, self.check_status)
        self.last_loss_sum = loss_sum
        if self.reduction == "sum":
            return costs.sum()
        if self.reduction == "mean":
            return costs.mean()
        return costs

    @torch.no_grad()
    def viterbi(self, emissions, predictions, input_lengths, label_lengths):
        """Best alignment with the label lengths given (teacher-forced predictions),
        as transducer/torch_binding.py:130-177.  Returns int32 [B, U]; entries past
        label_lengths[b] are unspecified padding."""
        device = emissions.device
        B, T, V = emissions.shape
        U = predictions.shape[1]
        labels = torch.empty((B, U - 1), device=device, dtype=torch.int32)
        certify_inputs(emissions, predictions, labels, input_lengths, label_lengths,
                       self.validate_lengths)
        emissions = emissions.contiguous()
        predictions = predictions.contiguous()
        with DeviceManager(device):
            nbytes = _transducer.viterbi_decode_workspace_bytes(B, T, U, V)
            ws = _workspace(nbytes, device)
            _transducer.viterbi_decode(
                emissions.data_ptr(), predictions.data_ptr(), input_lengths.data_ptr(),
                label_lengths.data_ptr(), labels.data_ptr(), B, T, U, V, self.blank,
                ws.data_ptr(), nbytes)
            if self.check_status:
                rc = _transducer.check_status()
                raise_for_status(rc, _transducer.last_error() if rc else "")
        return labels


def check_type(var, t, name):
    if var.dtype is not t:
        raise TypeError("{} must be {}".format(name, t))


def check_contiguous(var, name):
    if not var.is_contiguous():
        raise ValueError("{} must be contiguous".format(name))


def check_dim(var, dim, name):
    if len(var.shape) != dim:
        raise ValueError("{} must be {}D".format(name, dim))


def certify_inputs(emissions, predictions, labels, input_lengths, label_lengths,
                   validate_lengths=True, allow_bf16=False):
    """Argument checks with the reference's exception types and messages
    (transducer/torch_binding.py:195-229).  Dimensionality is checked first here so a
    wrong rank reports itself rather than an index error.  allow_bf16: emissions and
    predictions may both be bfloat16 instead of float32 (the loss; not in the reference)."""
    check_dim(emissions, 3, "emissions")
    check_dim(predictions, 3, "predictions")
    check_dim(labels, 2, "labels")
    check_dim(input_lengths, 1, "input_lengths")
    check_dim(label_lengths, 1, "label_lengths")
    if allow_bf16 and emissions.dtype is torch.bfloat16:
        check_type(predictions, torch.bfloat16, "predictions")
    else:
        check_type(emissions, torch.float32, "emissions")
        check_type(predictions, torch.float32, "predictions")
    check_type(labels, torch.int32, "labels")
    check_type(input_lengths, torch.int32, "input_lengths")
    check_type(label_lengths, torch.int32, "label_lengths")
    check_contiguous(labels, "labels")
    check_contiguous(label_lengths, "label_lengths")
    check_contiguous(input_lengths, "lengths")

    batch = emissions.shape[0]
    if emissions.shape[2] != predictions.shape[2]:
        raise ValueError("vocab size mismatch.")
    if input_lengths.shape[0] != batch:
        raise ValueError("must have a length per example.")
    if label_lengths.shape[0] != batch:
        raise ValueError("must have a label length per example.")
    if labels.shape[0] != batch:
        raise ValueError("must have a label per example.")
    if labels.shape[1] != (predictions.shape[1] - 1):
        raise ValueError("labels must be padded to maximum label length.")
    devices = {t.device for t in (emissions, predictions, labels, input_lengths, label_lengths)}
    if len(devices) != 1:
        raise ValueError("all inputs must be on the same device.")
    if batch == 0 or not validate_lengths:
        return
    # one device->host transfer for both maxima (the reference does two, :222-229)
    max_t, max_u = torch.stack((input_lengths.max(), label_lengths.max())).tolist()
    if emissions.shape[1] < max_t:
        raise ValueError("Input length mismatch")
    if predictions.shape[1] < max_u + 1:
        raise ValueError("Output length mismatch")
