"""Seeded synthetic workloads with the shapes, lengths and value distributions of the
benchmark configurations (stand-ins for the reference README's ``torch.rand``
benchmark shapes, benchmarks/torch_benchmarks.py:22-36; no external data).

Each utterance is drawn from its own seed, so any shard or subset of a batch can be
regenerated independently (a rank of a data-parallel run generates only its shard).
"""
from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    T: int
    U: int            # longest label sequence; predictions have U + 1 rows
    V: int
    std: float = 1.0
    t_range: tuple = None      # (lo, hi) inclusive for input_lengths; None = all T
    u_range: tuple = None      # (lo, hi) inclusive for label_lengths; None = all U
    peaky: float = 0.0         # fraction of entries per frame boosted by `boost`
    boost: float = 0.0
    blank_bias: float = 0.0    # added to the blank column of the emissions
    blank: int = 0
    task: str = "loss"         # "loss" (fwd+bwd), "loss_fwd" or "viterbi"
    extra: dict = field(default_factory=dict)


CONFIGS = {
    # CPU-runnable plumbing case
    "c1": Workload("c1", B=2, T=50, U=10, V=30, t_range=(25, 50), u_range=(1, 10)),
    # README shape, V swept
    "c2_v100": Workload("c2_v100", B=8, T=2000, U=100, V=100),
    "c2_v1000": Workload("c2_v1000", B=8, T=2000, U=100, V=1000),
    "c2_v2000": Workload("c2_v2000", B=8, T=2000, U=100, V=2000),
    "c2_v10000": Workload("c2_v10000", B=8, T=2000, U=100, V=10000),
    # large batch, single-GPU headline
    "c3": Workload("c3", B=32, T=2000, U=100, V=10000, std=2.0,
                   t_range=(1500, 2000), u_range=(60, 100)),
    # word-piece vocabulary, batch-sharded (loss only)
    "c4": Workload("c4", B=256, T=1000, U=200, V=32000, t_range=(500, 1000),
                   u_range=(100, 200), peaky=0.05, boost=6.0, task="loss_fwd"),
    # Viterbi best path
    "c5": Workload("c5", B=64, T=1500, U=150, V=4096, t_range=(750, 1500),
                   u_range=(75, 150), blank_bias=4.0, task="viterbi"),
    # not a benchmark configuration of the reference: the shape of c5 through the loss (forward +
    # backward), i.e. a label axis of more than 128 positions in the gradient kernels
    "c5_loss": Workload("c5_loss", B=64, T=1500, U=150, V=4096, t_range=(750, 1500),
                        u_range=(75, 150), blank_bias=4.0, task="loss"),
}


def _utt_seed(w, b):
    h = 1469598103934665603
    for ch in (w.name + ":%d" % b).encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h & 0x7FFFFFFFFFFFFFFF


def generate(w, device="cpu", first=0, count=None, force_full_first=True):
    """Tensors for utterances [first, first+count) of workload `w` on `device`:
    (emissions [n,T,V], predictions [n,U+1,V], labels [n,U] int32,
     input_lengths [n] int32, label_lengths [n] int32).

    Utterance 0 of the whole batch is forced to full length (as the reference's own
    random tests do, torch_test.py:181-182) so the padded shapes are tight."""
    count = w.B - first if count is None else count
    dev = torch.device(device)
    E = torch.empty((count, w.T, w.V), dtype=torch.float32, device=dev)
    P = torch.empty((count, w.U + 1, w.V), dtype=torch.float32, device=dev)
    labels = torch.empty((count, w.U), dtype=torch.int32)
    in_lens = torch.empty((count,), dtype=torch.int32)
    lab_lens = torch.empty((count,), dtype=torch.int32)
    for k in range(count):
        b = first + k
        seed = _utt_seed(w, b)
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        E[k].normal_(0.0, w.std, generator=g)
        P[k].normal_(0.0, w.std, generator=g)
        if w.peaky > 0.0:
            mask = torch.rand((w.T, w.V), generator=g, device=dev) < w.peaky
            E[k] += w.boost * mask
        if w.blank_bias != 0.0:
            E[k, :, w.blank] += w.blank_bias
        gc = torch.Generator()
        gc.manual_seed(seed ^ 0x5DEECE66D)
        lab = torch.randint(1, w.V, (w.U,), generator=gc, dtype=torch.int32)
        if w.blank != 0:
            lab = torch.where(lab == w.blank, torch.zeros_like(lab), lab)
        labels[k] = lab
        tl = w.T if w.t_range is None else int(torch.randint(w.t_range[0], w.t_range[1] + 1, (1,), generator=gc))
        ul = w.U if w.u_range is None else int(torch.randint(w.u_range[0], w.u_range[1] + 1, (1,), generator=gc))
        if force_full_first and b == 0:
            tl, ul = w.T, w.U
        in_lens[k] = tl
        lab_lens[k] = ul
    return E, P, labels.to(dev), in_lens.to(dev), lab_lens.to(dev)


def algorithmic_bytes(w, in_lens, lab_lens, elem_bytes=4):
    """HBM bytes the loss must move at minimum (emissions, predictions and gradients of
    elem_bytes each, fp32 lattices): forward reads E and P once over the valid rows and
    writes/reads the lattices; backward re-reads E and P, writes the full padded gradients and
    touches four lattices."""
    eb = float(elem_bytes)
    sum_t = float(in_lens.sum())
    sum_u = float((lab_lens + 1).sum())
    sum_tu = float((in_lens.double() * (lab_lens.double() + 1)).sum())
    n = len(in_lens)
    fwd = eb * w.V * (sum_t + sum_u) + 3 * 4.0 * sum_tu
    bwd = eb * w.V * (sum_t + sum_u) + eb * w.V * n * (w.T + w.U + 1) + 4 * 4.0 * sum_tu
    return {"fwd": fwd, "bwd": bwd, "total": fwd + bwd}


def algorithmic_flops(w, in_lens, lab_lens):
    """2*V per lattice node per contraction: one forward, two backward."""
    sum_tu = float((in_lens.double() * (lab_lens.double() + 1)).sum())
    return {"fwd": 2.0 * w.V * sum_tu, "bwd": 4.0 * w.V * sum_tu, "total": 6.0 * w.V * sum_tu}
