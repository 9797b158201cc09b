"""Generates the committed fixtures in this folder.  Run where the reference
checkout is available (it is NOT available where the GPU tests run):

    python tests/golden/make_golden.py /path/to/reference

1. reference_kats.json -- the literal known-answer vectors of the reference's own
   tests, read as text from transducer/test.cpp (smallTest :132-165, bigTest :167-226,
   viterbiTest :228-309; torch_test.py:41-158 repeats the same numbers) plus the
   analytic tinyTest (:92-130) evaluated in double precision.
2. reference_runs.npz -- seeded inputs pushed through the reference's CPU backend
   compiled unchanged from its sources (oracle/_ref/libref_transducer.so) together
   with the torch-op arithmetic of transducer/torch_binding.py, i.e. what
   TransducerLoss / criterion.viterbi return on CPU.
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402


def _function_body(src, name):
    start = src.index("void %s()" % name)
    depth, i = 0, src.index("{", start)
    begin = i
    while True:
        if src[i] == "{":
            depth += 1
        elif src[i] == "}":
            depth -= 1
            if depth == 0:
                return src[begin + 1:i]
        i += 1


def _vectors(body):
    out = {}
    for m in re.finditer(r"std::vector<(float|int)>\s+(\w+)\s*=\s*\{(.*?)\};", body, re.S):
        kind, name, nums = m.groups()
        vals = [x for x in re.split(r"[\s,]+", re.sub(r"//.*", "", nums)) if x]
        out[name] = [float(v) if kind == "float" else int(v) for v in vals]
    for m in re.finditer(r"int\s+(\w+)\s*=\s*(\d+);", body):
        out[m.group(1)] = int(m.group(2))
    m = re.search(r"float\s+expectedCost\s*=\s*([0-9.eE+-]+);", body)
    if m:
        out["expectedCost"] = float(m.group(1))
    return out


def kats_from_reference(ref_root):
    src = open(os.path.join(ref_root, "transducer", "test.cpp")).read()
    kats = {}

    s = _vectors(_function_body(src, "smallTest"))
    kats["small"] = dict(
        emissions=s["emissions"], predictions=s["predictions"], labels=s["labels"],
        input_lengths=[s["inputLength"]], label_lengths=[s["labelLength"]], V=s["alphabetSize"],
        costs=[s["expectedCost"]], egrads=s["expectedEgrads"], pgrads=s["expectedPgrads"])

    b = _vectors(_function_body(src, "bigTest"))
    kats["big"] = dict(
        emissions=b["emissions"], predictions=b["predictions"], labels=b["labels"],
        input_lengths=b["inputLengths"], label_lengths=b["labelLengths"], V=b["alphabetSize"],
        costs=b["expectedCosts"], egrads=b["expectedEgrads"], pgrads=b["expectedPgrads"])

    # tinyTest: T=2, U=0 labels, V=2; expectations are closed-form in the test itself
    e, p = [1.0, 2.0, 3.0, 4.0], [1.0, 2.0]
    ln1 = np.log(np.exp(e[0] + p[0]) + np.exp(e[1] + p[1]))
    ln2 = np.log(np.exp(e[2] + p[0]) + np.exp(e[3] + p[1]))
    eg = [np.exp(e[0] + p[0] - ln1) - 1, np.exp(e[1] + p[1] - ln1),
          np.exp(e[2] + p[0] - ln2) - 1, np.exp(e[3] + p[1] - ln2)]
    kats["tiny"] = dict(
        emissions=e, predictions=p, labels=[], input_lengths=[2], label_lengths=[0], V=2,
        costs=[float(-(e[0] + p[0] - ln1 + e[2] + p[0] - ln2))],
        egrads=[float(x) for x in eg], pgrads=[float(eg[0] + eg[2]), float(eg[1] + eg[3])])

    vb = _function_body(src, "viterbiTest")
    blocks = re.split(r"\{\s*//", vb)[1:]
    vit = []
    for blk in blocks:
        v = _vectors(blk)
        call = re.search(r"labelLengths\.data\(\),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),\s*(\d+),", blk)
        B, T, U, V, blank = (int(x) for x in call.groups())
        exp = re.search(r"checkSame\(labels,\s*\{([^}]*)\}\)", blk)
        vit.append(dict(
            title=blk.strip().splitlines()[0].strip(),
            emissions=v.get("emissions", []), predictions=v.get("predictions", []),
            input_lengths=v["inputLengths"], label_lengths=v["labelLengths"],
            B=B, T=T, U=U, V=V, blank=blank,
            labels=[int(x) for x in exp.group(1).split(",")] if exp else []))
    kats["viterbi"] = vit
    return kats


RUN_CASES = [
    # name, B, T, U' (=rows of predictions), V, std, zero_lengths
    ("c1", 2, 50, 11, 30, 1.0, False),
    ("ragged_zero", 3, 7, 4, 5, 1.0, True),
    ("v101", 6, 100, 10, 101, 1.0, True),
    ("no_labels", 4, 10, 1, 20, 1.0, False),
    ("v128", 2, 200, 33, 128, 1.0, False),
    ("v260_std2", 2, 150, 21, 260, 2.0, False),
    ("single", 1, 1, 1, 8, 1.0, False),
]


def reference_runs():
    assert O.have_reference(), "build oracle/_ref first: make -C oracle"
    out = {}
    for idx, (name, B, T, U, V, std, zero) in enumerate(RUN_CASES):
        rng = np.random.default_rng(1000 + idx)
        E = (std * rng.standard_normal((B, T, V))).astype(np.float32)
        P = (std * rng.standard_normal((B, U, V))).astype(np.float32)
        labels = rng.integers(1, V, (B, max(U - 1, 0))).astype(np.int32)
        lo_t = 0 if zero else max(1, T // 2)
        il = rng.integers(lo_t, T + 1, B).astype(np.int32)
        ll = rng.integers(0 if (zero or U == 1) else 1, U, B).astype(np.int32) if U > 1 \
            else np.zeros(B, np.int32)
        il[0], ll[0] = T, U - 1
        deltas = rng.uniform(0.5, 1.5, B).astype(np.float32)
        r = O.loss_and_grads(E, P, labels, il, ll, blank=0, deltas=deltas, impl="reference")
        vit = O.viterbi(E, P, il, ll, blank=0, impl="reference", fill=-1)
        for k, v in dict(E=E, P=P, labels=labels, in_lens=il, lab_lens=ll, deltas=deltas,
                         costs=r["costs"], egrads=r["egrads"], pgrads=r["pgrads"],
                         log_norms=r["log_norms"], viterbi=vit).items():
            out["%s/%s" % (name, k)] = v
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference/checkout")
    ref_root = sys.argv[1]
    kats = kats_from_reference(ref_root)
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(kats, f, indent=1)
    runs = reference_runs()
    np.savez_compressed(os.path.join(HERE, "reference_runs.npz"), **runs)
    print("wrote reference_kats.json (%d groups) and reference_runs.npz (%d arrays)"
          % (len(kats), len(runs)))


if __name__ == "__main__":
    main()
