"""Writes tests/golden/ref_util_tables.npz from the reference's own Python code.

The reference's ``kangaroo/util.py`` is Python 2 as a whole (an ``except A, B:`` further down),
but the part that defines the ordinal encoding -- the three 256-entry ``str.translate`` tables,
``acgtcomplement`` and ``revcomp`` (kangaroo/util.py:40-116) -- is plain code that Python 3
executes unchanged.  This script executes exactly that span of the file where it lies and stores
what it computes:

* ``acgt2ord``    [256] uint8: the ordinal every input byte is translated to,
* ``complement``  [256] uint8: the character every input byte is complemented to,
* ``ord2acgt``    [256] uint8: the character every ordinal is written back as,
* ``texts`` / ``revcomps``: sample strings (all cases, U, N, other bytes) and the reference's
  ``revcomp`` of each, newline-separated latin-1,
* ``b<k>_seqs``, ``b<k>_padding_rc``, ``b<k>_X``, ``b<k>_R``: sample minibatches and the ordinal
  buffer and region table the reference's batch-assembly statements (kangaroo/data.py:283-284,
  326-334) make of them, with and without reverse complements,
* ``strand_Z``, ``strand_kept``, ``strand_mask``: scores of forward / reverse-complement row pairs
  and what the reference's ``maskout_revcomp`` (kangaroo/predict.py:144-164) keeps of them.

Only ``acgt2ord``'s last step differs from the reference run: Python 3 strings have no buffer
interface, so the translated string is encoded to bytes (latin-1) instead of being wrapped by
``np.ndarray(buffer=...)``; the table is stored as it stands.

    python tests/golden/make_ref_util.py <reference root>
"""
import os
import sys

import numpy as np


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DEEPBIND_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_ref_util.py <reference root>")
    path = os.path.join(root, "code", "libs", "kangaroo", "kangaroo", "util.py")
    lines = open(path).read().splitlines()
    lo = next(i for i, l in enumerate(lines) if l.startswith("import numpy"))
    hi = next(i for i, l in enumerate(lines) if l.startswith("def str2intlist"))
    ns = {}
    exec(compile("\n".join(lines[lo:hi]), path, "exec"), ns)
    tab = lambda t: np.frombuffer(t.encode("latin-1"), np.uint8).copy()
    rng = np.random.Generator(np.random.PCG64(7))
    alphabet = "ACGTacgtUuNn.-XR*\xff\x00 "
    texts = ["".join(rng.choice(list(alphabet), size=int(n))) for n in rng.integers(1, 60, size=40)]
    texts += ["ACGT", "TTTT", "acgu", "N", "GATTACA"]
    revs = [ns["revcomp"](t) for t in texts]
    comps = [ns["acgtcomplement"](t) for t in texts]
    assert all("\n" not in t for t in texts)
    # Batch assembly: the statements of kangaroo/data.py that lay a minibatch out (``asbatches``,
    # data.py:326-334: region table, padded concatenation, encoding) and that interleave the
    # reverse complements (``_insert_reversecomplements``, data.py:283-284), taken from the file by
    # their text and executed on sample minibatches.  ``acgt2ord`` is the reference's translate()
    # with the Python 3 adaptation described above.
    dpath = os.path.join(root, "code", "libs", "kangaroo", "kangaroo", "data.py")
    dlines = [l.strip() for l in open(dpath).read().splitlines()]
    pick = lambda start: next(l for l in dlines if l.startswith(start))
    rc_stmts = [pick("rows = range(len(X))"), pick("Xrev = [acgtcomplement("), pick("newX = [Xrev[i] if j else X[i]")]
    asm_stmts = [pick("batchR = np.asarray(np.cumsum("), pick("batchR = np.hstack("), pick("batchX = acgt2ord((")]
    env = dict(ns)
    env["acgt2ord"] = lambda t: np.frombuffer(t.translate(ns["_acgt2ord"]).encode("latin-1"), np.uint8).reshape(1, -1)
    batches = {}
    for k, (padding, rc) in enumerate([(0, False), (15, False), (23, True), (11, True)]):
        seqs = ["".join(rng.choice(list("ACGTNacgu"), size=int(n))) for n in rng.integers(1, 50, size=9)]
        loc = dict(env, X=list(seqs), padding=padding)
        if rc:
            for st in rc_stmts:
                exec(st, loc)
            loc["batchX"] = loc["newX"]
        else:
            loc["batchX"] = list(seqs)
        for st in asm_stmts:
            exec(st, loc)
        batches["b%d_seqs" % k] = np.frombuffer("\n".join(seqs).encode("latin-1"), np.uint8)
        batches["b%d_padding_rc" % k] = np.array([padding, int(rc)])
        batches["b%d_X" % k] = np.asarray(loc["batchX"]).reshape(-1).copy()
        batches["b%d_R" % k] = np.asarray(loc["batchR"]).copy()
    # Strand selection at prediction time: the function maskout_revcomp of kangaroo/predict.py
    # (lines 144-164; the file as a whole is Python 2 because of print statements elsewhere),
    # executed as it stands with a stand-in for deepity's ``globals.flags`` and for ``np.bool``,
    # which NumPy has since removed.  Scores with ties, negatives, zeros of both signs.
    plines = open(os.path.join(root, "code", "libs", "kangaroo", "kangaroo", "predict.py")).read().splitlines()
    a = next(i for i, l in enumerate(plines) if l.startswith("def maskout_revcomp"))
    b = next(i for i in range(a + 1, len(plines)) if plines[i] and not plines[i][0].isspace())
    if not hasattr(np, "bool"):
        np.bool = bool
    flags = type("globals", (), {"flags": {"reverse_complement": True}})
    env2 = {"np": np, "globals": flags}
    exec(compile("\n".join(plines[a:b]), "predict.py", "exec"), env2)
    Z = rng.standard_normal((64, 1)).astype(np.float32)
    Z[4:8] = Z[4:8].round(1); Z[10] = Z[11]; Z[12], Z[13] = 0.0, -0.0; Z[14], Z[15] = -0.0, 0.0; Z[20] = Z[21] = -1.5
    kept, Zmask = env2["maskout_revcomp"](Z.copy())
    batches.update(strand_Z=Z, strand_kept=np.asarray(kept, np.float32), strand_mask=np.asarray(Zmask, bool))
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_util_tables.npz")
    np.savez_compressed(out, acgt2ord=tab(ns["_acgt2ord"]), complement=tab(ns["_acgtcomplement"]), ord2acgt=tab(ns["_ord2acgt"]),
                        texts=np.frombuffer("\n".join(texts).encode("latin-1"), np.uint8),
                        revcomps=np.frombuffer("\n".join(revs).encode("latin-1"), np.uint8),
                        complements=np.frombuffer("\n".join(comps).encode("latin-1"), np.uint8), **batches)
    print("wrote", out)


if __name__ == "__main__":
    main()
