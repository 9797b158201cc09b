"""Helpers that drive the library through its C ABI (ctypes on
libtransducer_b200.so) with device buffers held by torch tensors."""
import numpy as np
import torch

from transducer_b200 import _lib

lib = _lib.lib
check = _lib.check


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


def use_torch_stream():
    check(lib.tb200_set_stream(torch.cuda.current_stream().cuda_stream))


def set_option(key, value):
    check(lib.tb200_set_option(key.encode(), int(value)))


def shapes(E, P):
    B, T, V = E.shape
    return B, T, P.shape[1], V


def workspace(nbytes):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device="cuda")


def log_norms(E, P, il, ll):
    """tb200_log_norms -> (LN, rowRef, maxP) as device tensors (padding zeroed here)."""
    B, T, U, V = shapes(E, P)
    LN = torch.zeros((B, T, U), device="cuda")
    row_ref = torch.zeros((B, T), device="cuda")
    max_p = torch.zeros((B, U), device="cuda")
    n = lib.tb200_log_norms_workspace_bytes(B, T, U, V)
    ws = workspace(n)
    use_torch_stream()
    check(lib.tb200_log_norms(ptr(E), ptr(P), ptr(LN), ptr(row_ref), ptr(max_p), ptr(il), ptr(ll),
                              B, T, U, V, ptr(ws), n))
    return LN, row_ref, max_p


def forward(E, P, LN, labels, il, ll, blank=0):
    B, T, U, V = shapes(E, P)
    costs = torch.zeros((B,), device="cuda")
    alphas = torch.zeros((B, T, U), device="cuda")
    use_torch_stream()
    check(lib.tb200_forward(ptr(E), ptr(P), ptr(costs), ptr(alphas), ptr(LN), ptr(labels), ptr(il),
                            ptr(ll), B, T, U, V, blank))
    return costs, alphas


def backward(E, P, alphas, LN, labels, il, ll, blank=0):
    B, T, U, V = shapes(E, P)
    eg = torch.full((B, T, V), float("nan"), device="cuda")
    pg = torch.full((B, U, V), float("nan"), device="cuda")
    lg = torch.full((B, T, U), float("nan"), device="cuda")
    use_torch_stream()
    check(lib.tb200_backward(ptr(E), ptr(P), ptr(eg), ptr(pg), ptr(lg), ptr(alphas), ptr(LN),
                             ptr(labels), ptr(il), ptr(ll), B, T, U, V, blank))
    return eg, pg, lg


def viterbi(E, P, LN, il, ll, blank=0, fill=-1):
    B, T, U, V = shapes(E, P)
    out = torch.full((B, max(U - 1, 0)), fill, dtype=torch.int32, device="cuda")
    use_torch_stream()
    check(lib.tb200_viterbi(ptr(E), ptr(P), ptr(LN), ptr(out), ptr(il), ptr(ll), B, T, U, V, blank))
    return out


def loss_forward(E, P, labels, il, ll, blank=0):
    """tb200_loss_forward -> dict(costs, loss_sum, saved)."""
    B, T, U, V = shapes(E, P)
    out = dict(costs=torch.zeros((B,), device="cuda"), loss_sum=torch.zeros((1,), device="cuda"))
    ns = lib.tb200_loss_saved_bytes(B, T, U, V)
    out["saved"] = workspace(ns)
    n = lib.tb200_loss_forward_workspace_bytes(B, T, U, V)
    ws = workspace(n)
    use_torch_stream()
    fn = lib.tb200_loss_forward_bf16 if E.dtype == torch.bfloat16 else lib.tb200_loss_forward
    check(fn(ptr(E), ptr(P), ptr(labels), ptr(il), ptr(ll), ptr(out["costs"]),
             ptr(out["loss_sum"]), ptr(out["saved"]), ns, B, T, U, V, blank, ptr(ws), n))
    return out


def loss_backward(E, P, labels, il, ll, fwd, deltas=None, blank=0):
    B, T, U, V = shapes(E, P)
    eg = torch.full((B, T, V), float("nan"), device="cuda", dtype=E.dtype)
    pg = torch.full((B, U, V), float("nan"), device="cuda", dtype=E.dtype)
    if deltas is None:
        deltas = torch.ones((B,), device="cuda")
    n = lib.tb200_loss_backward_workspace_bytes(B, T, U, V)
    ws = workspace(n)
    use_torch_stream()
    fn = lib.tb200_loss_backward_bf16 if E.dtype == torch.bfloat16 else lib.tb200_loss_backward
    check(fn(ptr(E), ptr(P), ptr(labels), ptr(il), ptr(ll), ptr(fwd["saved"]),
             fwd["saved"].numel(), ptr(deltas), ptr(eg), ptr(pg), B, T, U, V, blank, ptr(ws), n))
    return eg, pg


def viterbi_decode(E, P, il, ll, blank=0, fill=-1):
    B, T, U, V = shapes(E, P)
    out = torch.full((B, max(U - 1, 0)), fill, dtype=torch.int32, device="cuda")
    n = lib.tb200_viterbi_decode_workspace_bytes(B, T, U, V)
    ws = workspace(n)
    use_torch_stream()
    check(lib.tb200_viterbi_decode(ptr(E), ptr(P), ptr(il), ptr(ll), ptr(out), B, T, U, V, blank,
                                   ptr(ws), n))
    return out


def label_arc_scores(E, P, il, ll, blank=0, fill=float("nan")):
    B, T, U, V = shapes(E, P)
    out = torch.full((B, T, U), fill, dtype=torch.float32, device="cuda")
    n = lib.tb200_label_arc_scores_workspace_bytes(B, T, U, V)
    ws = workspace(max(n, 256))
    use_torch_stream()
    check(lib.tb200_label_arc_scores(ptr(E), ptr(P), ptr(il), ptr(ll), ptr(out), B, T, U, V,
                                     blank, ptr(ws), n))
    return out


def case_to_device(c):
    """numpy case dict (E,P,labels,in_lens,lab_lens[,deltas]) -> device tensors."""
    d = dict(E=dev(c["E"]), P=dev(c["P"]), labels=dev(c["labels"], torch.int32),
             il=dev(c["in_lens"], torch.int32), ll=dev(c["lab_lens"], torch.int32))
    if "deltas" in c:
        d["deltas"] = dev(c["deltas"])
    return d


def rel_to_max(a, b):
    """max|a-b| / max|b| -- the gradient metric of the parity bar."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    den = np.abs(b).max() if b.size else 1.0
    return float(np.abs(a - b).max() / max(den, 1e-30)) if a.size else 0.0


def valid_mask(il, ll, T, U):
    il, ll = np.asarray(il), np.asarray(ll)
    m = np.zeros((len(il), T, U), bool)
    for b in range(len(il)):
        m[b, :il[b], :ll[b] + 1] = True
    return m
