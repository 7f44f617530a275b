"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (they stand in for the PBM / ChIP-seq / RNAcompete
datasets the reference trains on; no dataset record is reproduced).

Everything comes from ``numpy.random.Generator(PCG64(seed))``.  Sequences are
produced directly in the reference's batch layout
(code/libs/kangaroo/kangaroo/data.py:309-334): one uint8 buffer
``pad | s0 | pad | s1 | ... | pad`` with pad = m-1 bytes of 255, ordinals
A,C,G,T = 0..3, and a uint32 region table ``R[b] = (start of the leading pad of
sequence b, end of sequence b)``.
"""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def pack_batch(seqs, m):
    """List of uint8 ordinal arrays -> (X [npos] uint8, R [n,2] uint32)."""
    pad = m - 1
    lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=len(seqs))
    cum = np.concatenate([[0], np.cumsum(lens + pad)])
    X = np.full(int(cum[-1]) + pad, 255, np.uint8)
    for s, c in zip(seqs, cum[:-1]):
        X[c + pad:c + pad + len(s)] = s
    R = np.stack([cum[:-1], cum[1:]], axis=1).astype(np.uint32)
    return X, R


def uniform_batch(nseq, L, m, seed):
    """nseq sequences of equal length L, bases i.i.d. uniform over ACGT."""
    g = rng(seed)
    pad = m - 1
    bases = g.integers(0, 4, size=(nseq, L), dtype=np.uint8)
    buf = np.full((nseq, pad + L), 255, np.uint8)
    buf[:, pad:] = bases
    X = np.concatenate([buf.ravel(), np.full(pad, 255, np.uint8)])
    starts = np.arange(nseq, dtype=np.uint64) * (pad + L)
    R = np.stack([starts, starts + pad + L], axis=1).astype(np.uint32)
    return X, R


def revcomp_ord(s):
    """Reverse complement of an ordinal array; bytes outside 0..3 stay as they are
    (kangaroo/util.py:58-65,112-116 maps N to N)."""
    s = s[::-1].copy()
    acgt = s < 4
    s[acgt] = 3 - s[acgt]
    return s


def ragged_batch(nseq, lmin, lmax, m, seed, n_frac=0.0, both_strands=False):
    """Lengths uniform in [lmin, lmax]; a fraction n_frac of bases replaced by N (255).
    With both_strands the rows are interleaved fwd, rc, fwd, rc ... (data.py:274-283)."""
    g = rng(seed)
    lens = g.integers(lmin, lmax + 1, size=nseq)
    seqs = []
    for L in lens:
        s = g.integers(0, 4, size=int(L), dtype=np.uint8)
        if n_frac > 0:
            s[g.random(int(L)) < n_frac] = 255
        seqs.append(s)
        if both_strands:
            seqs.append(revcomp_ord(s))
    return pack_batch(seqs, m)


def model_params(nmodel, m, seed, pool="max", hidden=0, nmotif=16, wscale=0.05, dtype=np.float32):
    """Random-initialised weights of ``nmodel`` independent DeepBind models, laid
    out with the instance axis as the reference lays it out
    (corr1ord.py:57-58: filter columns instance-major; full.py:57: dense weights
    stacked on rows).  Filters N(0, wscale^2), motif bias U(-0.1, 0)."""
    g = rng(seed)
    I = nmodel
    npool = nmotif * (2 if pool == "all" else 1)
    p = {"Wscan": (g.standard_normal((4 * m, nmotif * I)) * wscale).astype(dtype),
         "bscan": g.uniform(-0.1, 0.0, size=nmotif * I).astype(dtype)}
    if hidden:
        p["W1"] = (g.standard_normal((npool * I, hidden)) * 0.1).astype(dtype)
        p["b1"] = (g.standard_normal(hidden * I) * 0.01).astype(dtype)
        p["W2"] = (g.standard_normal((hidden * I, 1)) * 0.1).astype(dtype)
        p["b2"] = (g.standard_normal(I) * 0.01).astype(dtype)
    else:
        p["W1"] = (g.standard_normal((npool * I, 1)) * 0.1).astype(dtype)
        p["b1"] = (g.standard_normal(I) * 0.01).astype(dtype)
    return p


CONFIGS = {
    # name: generator arguments of the five benchmark configurations
    "pbm_forward":   dict(nseq=4096, L=40, m=24, nmodel=1, pool="max", hidden=0),
    "chip_train":    dict(nseq=65536, L=101, m=24, nmodel=1, pool="all", hidden=32, batch=128),
    "calibration":   dict(nseq=20000, L=40, m=24, nmodel=90, pool="max", hidden=0, batch=64),
    "genome_scan":   dict(nseq=1000000, L=101, m=24, nmodel=512, pool="all", hidden=0),
    "ragged_rna":    dict(nseq=200000, lmin=20, lmax=200, m=16, nmodel=1, pool="max", hidden=0, n_frac=0.05),
}
