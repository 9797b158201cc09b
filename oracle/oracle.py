"""CPU oracle for the additive-joiner RNN-T loss / Viterbi path (TEST INFRASTRUCTURE).

Only tests/, the smoke check and bench.py's CPU legs import this module; the
product package never does.

Two backends sit behind the same functions:

* ``impl="port"``      -> ``liboracle.so`` built from ``oracle.c`` (the plain-C
  restatement of transducer/transducer_cpu.cpp);
* ``impl="reference"`` -> ``_ref/libref_transducer.so``, the reference's own CPU
  backend compiled unchanged from its sources by ``oracle/Makefile`` (its
  ``forward``/``backward``/``viterbi`` have C++ linkage, transducer/transducer.h:3-49,
  so they are bound by their mangled names).

A third library, ``_ref/libref_transducer_cuda.so``, is the reference's own CUDA backend
(transducer/transducer_cuda.cu) compiled unchanged for sm_100a; ``loss_and_grads_cuda``
runs the reference's whole GPU path with it: the GPU incumbent that bench.py can time and
a second checker for the GPU parity tests.

The arithmetic the reference does in torch ops around those three calls
(transducer/torch_binding.py:35-40 for the log-normalisers, :85-89 for the dense
part of the gradient, :162-167 for Viterbi) is restated here with the same torch
CPU ops in the same order, so ``loss_and_grads`` / ``viterbi`` reproduce what
``TransducerLoss`` returns on CPU.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libref_transducer.so")
_REF_CUDA_SO = os.path.join(_HERE, "_ref", "libref_transducer_cuda.so")

_f = ctypes.POINTER(ctypes.c_float)
_i = ctypes.POINTER(ctypes.c_int)
_c = ctypes.c_int

# mangled names of transducer.h's three functions (Itanium ABI)
_REF_FORWARD = "_Z7forwardPKfS0_PfS1_S0_PKiS3_S3_iiiiib"
_REF_BACKWARD = "_Z8backwardPKfS0_PfS1_S1_S0_S0_PKiS3_S3_iiiiib"
_REF_VITERBI = "_Z7viterbiPKfS0_S0_PiPKiS3_iiiiib"

_libs = {}


def build(quiet=True):
    """(Re)build liboracle.so and, where the reference sources exist, _ref/."""
    subprocess.run(["make", "-C", _HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def have_reference():
    return os.path.exists(_REF_SO)


def _port():
    if "port" not in _libs:
        if not os.path.exists(_PORT_SO):
            build()
        lib = ctypes.CDLL(_PORT_SO)
        lib.oracle_log_norms_exact.argtypes = [_f, _f, _f, _i, _i, _c, _c, _c, _c]
        lib.oracle_log_norms_factored.argtypes = [_f, _f, _f, _c, _c, _c, _c]
        lib.oracle_forward.argtypes = [_f, _f, _f, _f, _f, _i, _i, _i, _c, _c, _c, _c, _c]
        lib.oracle_backward.argtypes = [_f, _f, _f, _f, _f, _f, _f, _i, _i, _i, _c, _c, _c, _c, _c]
        lib.oracle_accumulate_grads_exact.argtypes = [_f, _f, _f, _f, _f, _f, _i, _i, _c, _c, _c, _c]
        lib.oracle_viterbi.argtypes = [_f, _f, _f, _i, _i, _i, _c, _c, _c, _c, _c]
        for fn in ("oracle_log_norms_exact", "oracle_log_norms_factored", "oracle_forward",
                   "oracle_backward", "oracle_accumulate_grads_exact", "oracle_viterbi"):
            getattr(lib, fn).restype = None
        _libs["port"] = lib
    return _libs["port"]


def _ref():
    if "ref" not in _libs:
        if not os.path.exists(_REF_SO):
            raise RuntimeError("reference CPU backend not built: run `make -C oracle` "
                               "where the reference sources are present")
        lib = ctypes.CDLL(_REF_SO)
        b = ctypes.c_bool
        fw = getattr(lib, _REF_FORWARD)
        fw.argtypes = [_f, _f, _f, _f, _f, _i, _i, _i, _c, _c, _c, _c, _c, b]
        bw = getattr(lib, _REF_BACKWARD)
        bw.argtypes = [_f, _f, _f, _f, _f, _f, _f, _i, _i, _i, _c, _c, _c, _c, _c, b]
        vt = getattr(lib, _REF_VITERBI)
        vt.argtypes = [_f, _f, _f, _i, _i, _i, _c, _c, _c, _c, _c, b]
        for fn in (fw, bw, vt):
            fn.restype = None
        _libs["ref"] = (fw, bw, vt)
    return _libs["ref"]


def _fp(a):
    return a.ctypes.data_as(_f) if a is not None and a.size else ctypes.cast(None, _f)


def _ip(a):
    return a.ctypes.data_as(_i) if a is not None and a.size else ctypes.cast(None, _i)


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _i32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


# ----------------------------------------------------------------------------
# the three transducer.h calls
# ----------------------------------------------------------------------------

def forward(E, P, LN, labels, in_lens, lab_lens, blank=0, impl="port"):
    """transducer.h:3-17 on host buffers -> (costs[B], alphas[B,T,U'])."""
    E, P, LN = _f32(E), _f32(P), _f32(LN)
    labels, in_lens, lab_lens = _i32(labels), _i32(in_lens), _i32(lab_lens)
    B, T, V = E.shape
    U = P.shape[1]
    costs = np.zeros(B, np.float32)
    alphas = np.zeros((B, T, U), np.float32)
    args = (_fp(E), _fp(P), _fp(costs), _fp(alphas), _fp(LN), _ip(labels), _ip(in_lens),
            _ip(lab_lens), B, T, U, V, blank)
    if impl == "reference":
        _ref()[0](*args, False)
    else:
        _port().oracle_forward(*args)
    return costs, alphas


def backward(E, P, alphas, LN, labels, in_lens, lab_lens, blank=0, impl="port"):
    """transducer.h:19-35 -> (egrads, pgrads, lngrads): zero-filled, sparse part only."""
    E, P, LN, alphas = _f32(E), _f32(P), _f32(LN), _f32(alphas)
    labels, in_lens, lab_lens = _i32(labels), _i32(in_lens), _i32(lab_lens)
    B, T, V = E.shape
    U = P.shape[1]
    eg = np.empty_like(E)
    pg = np.empty_like(P)
    lg = np.empty((B, T, U), np.float32)
    args = (_fp(E), _fp(P), _fp(eg), _fp(pg), _fp(lg), _fp(alphas), _fp(LN), _ip(labels),
            _ip(in_lens), _ip(lab_lens), B, T, U, V, blank)
    if impl == "reference":
        _ref()[1](*args, False)
    else:
        _port().oracle_backward(*args)
    return eg, pg, lg


def viterbi_abi(E, P, LN, in_lens, lab_lens, blank=0, impl="port", fill=-1):
    """transducer.h:37-49 -> labels[B,U'-1]; entries past label_lengths[b] keep `fill`."""
    E, P, LN = _f32(E), _f32(P), _f32(LN)
    in_lens, lab_lens = _i32(in_lens), _i32(lab_lens)
    B, T, V = E.shape
    U = P.shape[1]
    out = np.full((B, max(U - 1, 0)), fill, np.int32)
    args = (_fp(E), _fp(P), _fp(LN), _ip(out), _ip(in_lens), _ip(lab_lens), B, T, U, V, blank)
    if impl == "reference":
        _ref()[2](*args, False)
    else:
        _port().oracle_viterbi(*args)
    return out


# ----------------------------------------------------------------------------
# log-normalisers
# ----------------------------------------------------------------------------

def log_norms_exact(E, P, in_lens, lab_lens):
    """transducer/test.h:51-80: exact logsumexp per valid (t,u); padding is 0."""
    E, P = _f32(E), _f32(P)
    in_lens, lab_lens = _i32(in_lens), _i32(lab_lens)
    B, T, V = E.shape
    U = P.shape[1]
    LN = np.zeros((B, T, U), np.float32)
    _port().oracle_log_norms_exact(_fp(E), _fp(P), _fp(LN), _ip(in_lens), _ip(lab_lens), B, T, U, V)
    return LN


def log_norms_factored_c(E, P):
    """torch_binding.py:35-40 in plain C (index-order fp32 inner products)."""
    E, P = _f32(E), _f32(P)
    B, T, V = E.shape
    U = P.shape[1]
    LN = np.zeros((B, T, U), np.float32)
    _port().oracle_log_norms_factored(_fp(E), _fp(P), _fp(LN), B, T, U, V)
    return LN


def log_norms_torch(E, P):
    """torch_binding.py:35-40 with the same torch CPU ops; returns the pieces
    the reference keeps for its backward pass."""
    E = torch.as_tensor(np.asarray(E, np.float32))
    P = torch.as_tensor(np.asarray(P, np.float32))
    max_e = E.max(dim=2, keepdim=True)[0]
    max_p = P.max(dim=2, keepdim=True)[0]
    exp_e = torch.exp(E - max_e)
    exp_p = torch.exp(P - max_p)
    exp_ln = torch.bmm(exp_e, exp_p.transpose(1, 2))
    ln = torch.log(exp_ln) + max_e + max_p.transpose(1, 2)
    return ln, exp_e, exp_p, exp_ln


# ----------------------------------------------------------------------------
# the whole path, as TransducerLoss runs it on CPU
# ----------------------------------------------------------------------------

def loss_and_grads(E, P, labels, in_lens, lab_lens, blank=0, deltas=None, impl="port",
                   want_grads=True):
    """What ``TransducerLoss(blank)(E,P,labels,in_lens,lab_lens)`` followed by
    ``(deltas*costs).sum().backward()`` yields on CPU (torch_binding.py:25-90).

    Returns a dict with costs, alphas, log_norms and, if asked, egrads, pgrads,
    lngrads (the node occupancies)."""
    E, P = _f32(E), _f32(P)
    B = E.shape[0]
    ln_t, exp_e, exp_p, exp_ln = log_norms_torch(E, P)
    LN = ln_t.contiguous().numpy()
    costs, alphas = forward(E, P, LN, labels, in_lens, lab_lens, blank, impl)
    out = {"costs": costs, "alphas": alphas, "log_norms": LN}
    if not want_grads:
        return out
    eg, pg, lg = backward(E, P, alphas, LN, labels, in_lens, lab_lens, blank, impl)
    out["lngrads"] = lg.copy()
    d = torch.ones(B) if deltas is None else torch.as_tensor(np.asarray(deltas, np.float32))
    eg_t, pg_t = torch.from_numpy(eg), torch.from_numpy(pg)
    w = torch.from_numpy(lg) * exp_ln.reciprocal()
    eg_t += exp_e * torch.bmm(w, exp_p)
    pg_t += exp_p * torch.bmm(w.transpose(1, 2), exp_e)
    out["egrads"] = (d[:, None, None] * eg_t).numpy()
    out["pgrads"] = (d[:, None, None] * pg_t).numpy()
    return out


def viterbi(E, P, in_lens, lab_lens, blank=0, impl="port", fill=-1):
    """``TransducerLoss(blank).viterbi`` on CPU (torch_binding.py:130-177)."""
    ln_t = log_norms_torch(E, P)[0]
    return viterbi_abi(E, P, ln_t.contiguous().numpy(), in_lens, lab_lens, blank, impl, fill)


def accumulate_grads_exact(E, P, egrads, pgrads, lngrads, LN, in_lens, lab_lens):
    """transducer/test.h:82-113, in place on egrads/pgrads (small cases)."""
    E, P, LN, lngrads = _f32(E), _f32(P), _f32(LN), _f32(lngrads)
    in_lens, lab_lens = _i32(in_lens), _i32(lab_lens)
    B, T, V = E.shape
    U = P.shape[1]
    assert egrads.dtype == np.float32 and egrads.flags.c_contiguous
    assert pgrads.dtype == np.float32 and pgrads.flags.c_contiguous
    _port().oracle_accumulate_grads_exact(_fp(E), _fp(P), _fp(egrads), _fp(pgrads), _fp(lngrads),
                                          _fp(LN), _ip(in_lens), _ip(lab_lens), B, T, U, V)


# ----------------------------------------------------------------------------
# float64 "truth": the same loss by an alpha/beta recursion in double precision.
# Used only to attribute differences between two fp32 implementations to the
# fp32 noise floor of the recursion (alphas reach ~1e4 at T=2000, ulp ~1e-3).
# ----------------------------------------------------------------------------

def _alpha_beta64(stay, step):
    """float64 alpha and beta lattices [T,U] from the arc log-probabilities stay[t,u] (blank arc
    leaving (t,u)) and step[t,u] (label arc leaving (t,u); -inf in the last column), swept one
    anti-diagonal per numpy operation."""
    T, U = stay.shape
    D = T + U - 1
    ninf = -np.inf
    # skewed copies: X[d, u] = x[d - u, u]
    def skew(x):
        out = np.full((D, U), ninf)
        for u in range(U):
            out[u:u + T, u] = x[:, u]
        return out
    st, sp = skew(stay), skew(step)
    valid = np.isfinite(skew(np.zeros((T, U))))
    A = np.full((D, U), ninf)
    A[0, 0] = 0.0
    for d in range(1, D):
        from_stay = A[d - 1] + st[d - 1]                       # (t-1,u) -> (t,u)
        from_step = np.full(U, ninf)
        from_step[1:] = A[d - 1, :-1] + sp[d - 1, :-1]         # (t,u-1) -> (t,u)
        with np.errstate(invalid="ignore"):
            row = np.logaddexp(from_stay, from_step)
        A[d] = np.where(valid[d], row, ninf)
    Bt = np.full((D, U), ninf)
    Bt[D - 1, U - 1] = stay[T - 1, U - 1]
    for d in range(D - 2, -1, -1):
        to_stay = Bt[d + 1] + st[d]                            # (t,u) -> (t+1,u)
        to_step = np.full(U, ninf)
        to_step[:-1] = Bt[d + 1, 1:] + sp[d, :-1]              # (t,u) -> (t,u+1)
        with np.errstate(invalid="ignore"):
            row = np.logaddexp(to_stay, to_step)
        Bt[d] = np.where(valid[d], row, ninf)
    def unskew(X):
        out = np.empty((T, U))
        for u in range(U):
            out[:, u] = X[u:u + T, u]
        return out
    return unskew(A), unskew(Bt)


def truth64(E, P, labels, in_lens, lab_lens, blank=0):
    E = torch.as_tensor(np.asarray(E, np.float64))
    P = torch.as_tensor(np.asarray(P, np.float64))
    labels = np.asarray(labels)
    B, Tm, V = E.shape
    Um = P.shape[1]
    me = E.max(dim=2, keepdim=True)[0]
    mp = P.max(dim=2, keepdim=True)[0]
    xe, xp = torch.exp(E - me), torch.exp(P - mp)
    s = torch.bmm(xe, xp.transpose(1, 2))
    LN = (torch.log(s) + me + mp.transpose(1, 2)).numpy()
    En, Pn = E.numpy(), P.numpy()
    costs = np.full(B, np.inf)
    eg = np.zeros((B, Tm, V))
    pg = np.zeros((B, Um, V))
    for b in range(B):
        T, U = int(in_lens[b]), int(lab_lens[b]) + 1
        if T == 0 or U == 0:
            continue
        lab = labels[b, :U - 1].astype(np.int64)
        ln = LN[b, :T, :U]
        stay = En[b, :T, blank][:, None] + Pn[b, :U, blank][None, :] - ln          # [T,U]
        step = np.full((T, U), -np.inf)
        if U > 1:
            step[:, :U - 1] = En[b, :T][:, lab] + Pn[b, np.arange(U - 1), lab][None, :] - ln[:, :U - 1]
        al, be = _alpha_beta64(stay, step)
        ll = be[0, 0]
        costs[b] = -ll
        g = np.exp(al + be - ll)                                   # node occupancy
        occ_stay = np.zeros((T, U))
        occ_stay[:T - 1] = np.exp(al[:T - 1] + stay[:T - 1] + be[1:] - ll)
        occ_stay[T - 1, U - 1] = 1.0
        occ_step = np.zeros((T, U))
        if U > 1:
            occ_step[:, :U - 1] = np.exp(al[:, :U - 1] + step[:, :U - 1] + be[:, 1:] - ll)
        w = torch.from_numpy(g / s[b, :T, :U].numpy())
        eg[b, :T] = (xe[b, :T] * (w @ xp[b, :U])).numpy()
        pg[b, :U] = (xp[b, :U] * (w.T @ xe[b, :T])).numpy()
        eg[b, :T, blank] -= occ_stay.sum(1)
        pg[b, :U, blank] -= occ_stay.sum(0)
        for u in range(U - 1):
            eg[b, :T, lab[u]] -= occ_step[:, u]
            pg[b, u, lab[u]] -= occ_step[:, u].sum()
    return {"costs": costs, "egrads": eg, "pgrads": pg, "log_norms": LN}


# ----------------------------------------------------------------------------
# the reference's GPU path (its CUDA backend + the torch CUDA ops of its wrapper)
# ----------------------------------------------------------------------------

def have_reference_cuda():
    return os.path.exists(_REF_CUDA_SO)


def _ref_cuda():
    if "ref_cuda" not in _libs:
        if not have_reference_cuda():
            raise RuntimeError("reference CUDA backend not built: run `make -C oracle` "
                               "where the reference sources and nvcc are present")
        lib = ctypes.CDLL(_REF_CUDA_SO)
        v, b = ctypes.c_void_p, ctypes.c_bool
        fw = getattr(lib, _REF_FORWARD)
        fw.argtypes = [v] * 8 + [_c] * 5 + [b]
        bw = getattr(lib, _REF_BACKWARD)
        bw.argtypes = [v] * 10 + [_c] * 5 + [b]
        vt = getattr(lib, _REF_VITERBI)
        vt.argtypes = [v] * 6 + [_c] * 5 + [b]
        for fn in (fw, bw, vt):
            fn.restype = None
        _libs["ref_cuda"] = (fw, bw, vt)
    return _libs["ref_cuda"]


def loss_and_grads_cuda(E, P, labels, in_lens, lab_lens, blank=0, deltas=None,
                        want_grads=True):
    """``TransducerLoss`` of the reference on CUDA tensors (torch_binding.py:25-90):
    the same torch ops in the same order, on the device, around the reference's own
    forward/backward kernels (transducer_cuda.cu:280-348).  Those kernels are launched on
    the legacy default stream (transducer_cuda.cu:294,334), so the torch ops are put there
    too.  float32 E [B,T,V], P [B,U',V]; int32 labels [B,U'-1], lengths [B]; all on one
    CUDA device.  Returns a dict of device tensors."""
    fw, bw, _ = _ref_cuda()
    dev = E.device
    B, T, V = E.shape
    U = P.shape[1]
    with torch.cuda.device(dev), torch.cuda.stream(torch.cuda.default_stream(dev)):
        costs = torch.empty((B,), device=dev, dtype=torch.float32)
        alphas = torch.empty((B, T, U), device=dev, dtype=torch.float32)
        max_e = E.max(dim=2, keepdim=True)[0]
        max_p = P.max(dim=2, keepdim=True)[0]
        exp_e = torch.exp(E - max_e)
        exp_p = torch.exp(P - max_p)
        exp_ln = torch.bmm(exp_e, exp_p.transpose(1, 2))
        ln = torch.log(exp_ln) + max_e + max_p.transpose(1, 2)
        fw(E.data_ptr(), P.data_ptr(), costs.data_ptr(), alphas.data_ptr(), ln.data_ptr(),
           labels.data_ptr(), in_lens.data_ptr(), lab_lens.data_ptr(), B, T, U, V, blank, True)
        out = {"costs": costs, "alphas": alphas, "log_norms": ln}
        if not want_grads:
            return out
        eg = torch.empty((B, T, V), device=dev, dtype=torch.float32)
        pg = torch.empty((B, U, V), device=dev, dtype=torch.float32)
        lg = torch.empty((B, T, U), device=dev, dtype=torch.float32)
        bw(E.data_ptr(), P.data_ptr(), eg.data_ptr(), pg.data_ptr(), lg.data_ptr(),
           alphas.data_ptr(), ln.data_ptr(), labels.data_ptr(), in_lens.data_ptr(),
           lab_lens.data_ptr(), B, T, U, V, blank, True)
        d = torch.ones((B,), device=dev) if deltas is None else deltas
        lg = lg * exp_ln.reciprocal()
        eg += exp_e * torch.bmm(lg, exp_p)
        pg += exp_p * torch.bmm(lg.transpose(1, 2), exp_e)
        out["egrads"] = d[:, None, None] * eg
        out["pgrads"] = d[:, None, None] * pg
    return out


def viterbi_cuda(E, P, in_lens, lab_lens, blank=0, fill=-1):
    """``TransducerLoss.viterbi`` of the reference on CUDA tensors
    (torch_binding.py:130-177, transducer_cuda.cu:350-388)."""
    _, _, vt = _ref_cuda()
    dev = E.device
    B, T, V = E.shape
    U = P.shape[1]
    with torch.cuda.device(dev), torch.cuda.stream(torch.cuda.default_stream(dev)):
        max_e = E.max(dim=2, keepdim=True)[0]
        max_p = P.max(dim=2, keepdim=True)[0]
        exp_ln = torch.bmm(torch.exp(E - max_e), torch.exp(P - max_p).transpose(1, 2))
        ln = torch.log(exp_ln) + max_e + max_p.transpose(1, 2)
        labels = torch.full((B, max(U - 1, 0)), fill, device=dev, dtype=torch.int32)
        vt(E.data_ptr(), P.data_ptr(), ln.data_ptr(), labels.data_ptr(), in_lens.data_ptr(),
           lab_lens.data_ptr(), B, T, U, V, blank, True)
    return labels
