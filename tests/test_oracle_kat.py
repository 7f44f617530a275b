"""Known-answer tests that pin the CPU oracle.

The reference has no golden vectors for this path, so every expectation here is
derived by hand (or by an independent few-line restatement) from the kernel
sources cited in oracle/deepbind_oracle.c.
"""
import numpy as np
import pytest

f32 = np.float32


def onehot_filter(motif, nf=1, col=0):
    m = len(motif)
    W = np.zeros((4 * m, nf), f32)
    for j, ch in enumerate(motif):
        W[4 * j + "ACGT".index(ch), col] = 1
    return W


def test_asbatch_layout(orc):
    X, R = orc.asbatch(["ACGT", "GG"], 2)
    assert X.tolist() == [255, 255, 0, 1, 2, 3, 255, 255, 2, 2, 255, 255]
    assert R.tolist() == [[0, 6], [6, 10]]
    assert R.dtype == np.uint32 and X.dtype == np.uint8


def test_acgt2ord_and_revcomp(orc):
    assert orc.acgt2ord("ACGTUacgtuN.x").tolist() == [0, 1, 2, 3, 3, 0, 1, 2, 3, 3, 255, 255, 255]
    assert orc.revcomp("ATTGC") == "GCAAT"
    assert orc.revcomp("ANC") == "GNT"
    X, R = orc.asbatch(["AAC"], 1, reverse_complement=True)
    assert X.tolist() == [255, 0, 0, 1, 255, 2, 3, 3, 255]
    assert R.tolist() == [[0, 4], [4, 8]]


def test_scan_counts_matches_of_a_kmer_detector(orc):
    # Z[i] = number of window bases equal to the motif + 1/4 per padding byte.
    W = onehot_filter("ACGT")
    X, R = orc.asbatch(["TTACGTAA"], 3)
    Z = orc.corr1ord(W, X)
    seq = "...TTACGTAA..."
    want = []
    for i in range(len(seq) - 3):
        want.append(sum(0.25 if c == "." else float(c == mch) for c, mch in zip(seq[i:i + 4], "ACGT")))
    assert Z[:len(want), 0].tolist() == want
    assert Z[5, 0] == 4.0                       # window aligned with the motif
    assert np.all(Z[len(want):] == 0)           # last m-1 rows are left as they were


def test_scan_all_N_is_sum_of_tap_means(orc):
    rng = np.random.default_rng(1)
    m, nf = 5, 3
    W = rng.standard_normal((4 * m, nf)).astype(f32)
    X = np.full(9, 255, np.uint8)
    Z = orc.corr1ord(W, X)
    want = np.zeros(nf, f32)
    for j in range(m):
        t = W[4 * j] + W[4 * j + 1]
        t = t + W[4 * j + 2]
        t = t + W[4 * j + 3]
        want = want + t * f32(0.25)
    for i in range(9 - m + 1):
        assert np.array_equal(Z[i], want)


def test_scan_dropped_base_adds_nothing_and_tail_untouched(orc):
    W = onehot_filter("AAAA")
    X = np.array([0, 254, 0, 0, 0, 254, 254], np.uint8)
    Z = np.full((7, 1), -7.0, f32)
    orc.corr1ord(W, X, Z)
    assert Z[:4, 0].tolist() == [3.0, 3.0, 3.0, 2.0]
    assert Z[4:, 0].tolist() == [-7.0] * 3


def test_scan_accumulates_taps_in_ascending_order(orc):
    # ((1e8 + 1) - 1e8) differs from (1e8 + (1 - 1e8)) in float32.
    W = np.zeros((12, 1), f32)
    W[0, 0], W[4, 0], W[8, 0] = 1e8, 1.0, -1e8
    Z = orc.corr1ord(W, np.zeros(3, np.uint8))
    assert Z[0, 0] == f32(f32(f32(1e8) + f32(1.0)) - f32(1e8)) == 0.0


def test_scan_sequence_shorter_than_filter(orc):
    W = onehot_filter("ACGTAC")
    X, R = orc.asbatch(["CG"], 5)
    Z = orc.corr1ord(W, X)
    assert X.size == 12 and R.tolist() == [[0, 7]]
    # window at row 4 covers ".CG..." : taps 1,2 match, 4 pads
    assert Z[4, 0] == 2 + 4 * 0.25
    P, A = orc.poolrgn(Z, R, "max", True)
    assert P[0, 0] == 3.0 and A[0, 0] == 4


def test_pool_first_maximum_wins_and_flat_index(orc):
    U = np.array([[0, 5], [2, 5], [2, 1], [0, 9], [7, 9]], f32)
    R = np.array([[0, 3], [3, 5]], np.uint32)
    P, A = orc.poolrgn(U, R, "max", True)
    assert P.tolist() == [[2, 5], [7, 9]]
    assert A.tolist() == [[1 * 2 + 0, 0 * 2 + 1], [4 * 2 + 0, 3 * 2 + 1]]


def test_pool_all_interleaves_max_and_mean(orc):
    U = np.array([[1, 10], [3, 30], [2, 20]], f32)
    R = np.array([[0, 3]], np.uint32)
    P, A = orc.poolrgn(U, R, "all", True)
    assert P.tolist() == [[3, 2, 30, 20]]
    assert A.tolist() == [[2, 3]]
    Ps, _ = orc.poolrgn(U, R, "sum")
    assert Ps.tolist() == [[6, 60]]


def test_pool_step_column_uses_integer_count(orc):
    U = np.arange(7, dtype=f32).reshape(7, 1)
    R = np.array([[0, 7, 3]], np.uint32)          # rows 0,3,6 -> count (7+2)//3 = 3
    P, _ = orc.poolrgn(U, R, "avg")
    assert P[0, 0] == f32(9.0) / f32(3.0)
    R2 = np.array([[1, 6, 2]], np.uint32)         # rows 1,3,5 -> count (5+1)//2 = 3
    P2, A2 = orc.poolrgn(U, R2, "all", True)
    assert P2.tolist() == [[5, 3]] and A2.tolist() == [[5]]


def test_all_zero_maps_pick_first_row_of_region(orc):
    W = onehot_filter("ACGT", nf=2)
    X, R = orc.asbatch(["ACGTACGT", "TTTT"], 3)
    bias = np.array([-100, -100], f32)
    P, A = orc.scanpool(W, bias, True, X, R, "max", True)
    assert np.all(P == 0)
    assert A.tolist() == [[0 * 2, 0 * 2 + 1], [11 * 2, 11 * 2 + 1]]


def test_fused_equals_chain(orc):
    rng = np.random.default_rng(3)
    m, nf = 6, 5
    W = (rng.standard_normal((4 * m, nf)) * 0.3).astype(f32)
    b = rng.uniform(-0.3, 0, nf).astype(f32)
    seqs = ["".join(rng.choice(list("ACGTN"), size=n)) for n in (9, 3, 17, 6, 1)]
    X, R = orc.asbatch(seqs, m - 1)
    Z = orc.corr1ord(W, X)
    Aact = np.maximum(Z + b, 0)
    for pt in ("max", "avg", "sum", "all"):
        P, A = orc.poolrgn(Aact, R, pt, True)
        P2, A2 = orc.scanpool(W, b, True, X, R, pt, True)
        assert np.array_equal(P, P2)
        if A is not None:
            assert np.array_equal(A, A2)


def test_pool_bprop_all(orc):
    R = np.array([[0, 2], [2, 5]], np.uint32)
    P = np.array([[10, 4], [20, 9]], f32)         # (max delta, mean delta) pairs, one map
    A = np.array([[1], [2]], np.uint32)
    U = np.zeros((5, 1), f32)
    orc.poolrgn_bprop(U, R, P, A, "all")
    assert U[:, 0].tolist() == [2, 12, 23, 3, 3]


def test_bprop_W_and_X_against_definitions(orc):
    rng = np.random.default_rng(5)
    m, nf, n = 3, 2, 8
    W = rng.standard_normal((4 * m, nf))
    X = np.array([0, 1, 255, 3, 254, 2, 2, 1], np.uint8)
    dZ = rng.standard_normal((n, nf))
    dZ[n - m + 1:] = 0
    # dW by finite differences of sum(Z*dZ) in float64
    dW = orc.corr1ord_bprop_W(np.zeros_like(W), X, dZ)
    num = np.zeros_like(W)
    for idx in np.ndindex(*W.shape):
        Wp, Wm = W.copy(), W.copy()
        Wp[idx] += 1e-6; Wm[idx] -= 1e-6
        num[idx] = ((orc.corr1ord(Wp, X) - orc.corr1ord(Wm, X)) * dZ).sum() / 2e-6
    np.testing.assert_allclose(dW, num, rtol=1e-6, atol=1e-8)
    # dX from its defining sum (corr1ord_bprop.cu:191-201)
    dX = orc.corr1ord_bprop_X(np.zeros((n, 4)), W, dZ)
    want = np.zeros((n, 4))
    for i in range(n):
        for f in range(nf):
            for k in range(min(m, i + 1)):
                for c in range(4):
                    want[i, c] += dZ[i - k, f] * W[4 * k + c, f]
    np.testing.assert_allclose(dX, want, rtol=1e-12)


def test_gradstep_variants(orc):
    P = np.array([1.0, 2.0], f32); dP = np.array([0.5, -1.0], f32)
    dr = np.array([0.1, 0.2], f32); mP = np.array([1.0, 1.0], f32); mr = np.array([0.9, 0.5], f32)
    p, m_ = P.copy(), mP.copy()
    orc.gradstep(p, dP, dr, m_, mr)
    assert np.allclose(m_, [0.9 - 0.05, 0.5 + 0.2]) and np.allclose(p, [1 + 0.85, 2 + 0.7])
    p, m_ = P.copy(), mP.copy()
    orc.gradstep_nesterov1(p, m_, mr)
    assert np.allclose(p, [1.9, 2.5]) and np.array_equal(m_, mP)
    orc.gradstep_nesterov2(p, dP, dr, m_, mr)
    assert np.allclose(m_, [0.85, 0.7]) and np.allclose(p, [1.9 - 0.05, 2.5 + 0.2])


def test_madd_bcast_indexing(orc):
    A = np.ones(12, f32); dst = np.zeros(12, f32)
    orc.madd_bcast(A, np.array([1, 2, 3], f32), 2, dst)      # b[(i/2) % 3]
    assert dst.tolist() == [1, 1, 2, 2, 3, 3, 1, 1, 2, 2, 3, 3]


def test_zmask_tie_goes_to_forward_strand(orc):
    Z = np.array([[1.0], [1.0], [0.0], [2.0]], f32)
    M = np.zeros((4, 1), np.uint8)
    orc.calc_zmask(Z, M)
    assert M[:, 0].tolist() == [1, 0, 0, 1]
    S = orc.score_net.__doc__ is not None
    assert S


def test_dropout_semantics(orc):
    X = np.arange(1, 9, dtype=f32).reshape(2, 4)
    rate = np.array([0.5, 0.25], f32)             # two models, 2 columns each
    U = np.array([0.5, 0.49, 0.25, 0.2, 0.9, 0.1, 0.3, 0.26], f32)
    Z, M = orc.dropout_fp_tr(X, rate, U)
    assert M.ravel().tolist() == [True, False, True, False, True, False, True, True]
    assert np.array_equal(Z, X * M)               # no 1/(1-p) rescale at train time
    Zm, Mm = orc.dropout_fp_tr(X, rate, U[:4], matchrows=True)
    assert np.array_equal(Mm[0], Mm[1]) and Mm[0].tolist() == [True, False, True, False]
    assert np.allclose(orc.dropout_fp_te(X, rate), X * np.array([0.5, 0.5, 0.75, 0.75], f32))
    xo = np.array([0, 255, 3, 2], np.uint8)
    Zo, Mo = orc.dropoutord_fp_tr(xo, np.array([0.1, 0.1, 0.6, 0.5], f32), 0.5)
    assert Zo.tolist() == [254, 255, 3, 2] and Mo.tolist() == [False, True, True, True]


def test_blockwise_dots_match_per_block_matmul(orc):
    rng = np.random.default_rng(7)
    I, n, k, m = 3, 5, 4, 2
    X = rng.standard_normal((n, k * I)); W = rng.standard_normal((k * I, m)); dZ = rng.standard_normal((n, m * I))
    Z = orc.blockwise_dot(X, W, I)
    dX = orc.blockwise_dot_nt(dZ, W, I)
    dW = orc.blockwise_dot_tn(X, dZ, I, W)
    for b in range(I):
        Xb, Wb, dZb = X[:, b * k:(b + 1) * k], W[b * k:(b + 1) * k], dZ[:, b * m:(b + 1) * m]
        np.testing.assert_allclose(Z[:, b * m:(b + 1) * m], Xb @ Wb, rtol=1e-12)
        np.testing.assert_allclose(dX[:, b * k:(b + 1) * k], dZb @ Wb.T, rtol=1e-12)
        np.testing.assert_allclose(dW[b * k:(b + 1) * k], Xb.T @ dZb, rtol=1e-12)
    # shared input
    Xs = rng.standard_normal((n, k))
    Zs = orc.blockwise_dot(Xs, W, I)
    for b in range(I):
        np.testing.assert_allclose(Zs[:, b * m:(b + 1) * m], Xs @ W[b * k:(b + 1) * k], rtol=1e-12)
    # combined: two inputs stacked on the weight rows of each block
    X0 = rng.standard_normal((n, 3 * I)); X1 = rng.standard_normal((n, 1 * I))
    Zc = orc.blockwise_dot_combined([X0, X1], W, I, [False, False])
    for b in range(I):
        Wb = W[b * 4:(b + 1) * 4]
        want = X0[:, 3 * b:3 * b + 3] @ Wb[:3] + X1[:, b:b + 1] @ Wb[3:]
        np.testing.assert_allclose(Zc[:, b * m:(b + 1) * m], want, rtol=1e-12)


def test_train_grads_match_finite_differences(orc):
    # the whole training graph in float64, as deepity/gradcheck.py does for the reference
    from deepbind_b200 import synth
    rng = np.random.default_rng(11)
    I, m = 2, 5
    params = synth.model_params(I, m, 3, pool="all", hidden=4, nmotif=16, wscale=0.3, dtype=np.float64)
    seqs = ["".join(rng.choice(list("ACGT"), size=n)) for n in (9, 12, 7, 10)]
    X, R = orc.asbatch(seqs, m - 1)
    Y = rng.integers(0, 2, size=(4, 1)).astype(np.float64)
    mask = (rng.random((4, 32 * I)) > 0.3).astype(np.float64)
    for loss in ("nll", "mse"):
        L, g = orc.train_grads(params, X, R, Y, "all", I, loss, mask)
        for name in params:
            flat = params[name].ravel()
            for idx in rng.choice(flat.size, size=min(6, flat.size), replace=False):
                old = flat[idx]
                flat[idx] = old + 1e-6; Lp, _ = orc.train_grads(params, X, R, Y, "all", I, loss, mask)
                flat[idx] = old - 1e-6; Lm, _ = orc.train_grads(params, X, R, Y, "all", I, loss, mask)
                flat[idx] = old
                num = (Lp.sum() - Lm.sum()) / 2e-6
                assert abs(num - g[name].ravel()[idx]) <= 1e-6 + 1e-4 * abs(num), (loss, name, idx)


def test_strand_max_keeps_forward_on_ties(orc):
    from deepbind_b200 import synth
    m = 4
    p = synth.model_params(1, m, 5, pool="max", hidden=0)
    X, R = orc.asbatch(["ACGT"], m - 1, reverse_complement=True)   # palindrome: both strands equal
    s = orc.score_net(p, X, R, "max", 1, strand_max=True)
    both = orc.score_net(p, X, R, "max", 1)
    assert both[0, 0] == both[1, 0] == s[0, 0]


def test_scan_mode_windows(orc):
    """predict.py:281-284: W-1 'N' on both sides, every stride-th window of W characters."""
    assert orc.scan_windows("ACGT", 3) == ["NNA", "NAC", "ACG", "CGT", "GTN", "TNN"]
    assert orc.scan_windows("ACGT", 3, stride=4) == ["NNA", "GTN"]
    assert orc.scan_windows("A", 1) == ["A"]
    assert orc.scan_windows("", 3) == ["NNN", "NNN"]            # len(padseq) - W + 1 = 2 starts
    from deepbind_b200 import fused
    for L, W, s in [(4, 3, 1), (4, 3, 4), (1, 1, 1), (0, 3, 1), (37, 20, 7), (5, 64, 64)]:
        assert int(fused.window_counts([L], W, s)[0]) == len(orc.scan_windows("A" * L, W, s))


def test_input_gradients_against_finite_differences(orc):
    """dX of the gradient-map chain = d(1/2 sum Z^2)/d(one-hot input), checked with central
    differences on a dense float64 restatement (one-hot input times the filter taps)."""
    rng = np.random.default_rng(12)
    m, nf, L, nseq = 4, 16, 9, 3
    pad = m - 1
    seqs = [rng.integers(0, 4, L) for _ in range(nseq)]
    X = np.concatenate([np.concatenate([np.full(pad, 255, np.uint8), s.astype(np.uint8)]) for s in seqs] + [np.full(pad, 255, np.uint8)])
    R = np.array([[i * (L + pad), (i + 1) * (L + pad)] for i in range(nseq)], np.uint32)
    p = {"Wscan": rng.standard_normal((4 * m, nf)) * 0.5, "bscan": rng.uniform(-0.2, 0.2, nf),
         "W1": rng.standard_normal((nf, 1)), "b1": rng.standard_normal(1)}
    Z, dX = orc.input_gradients(p, X, R, "max", 1, "mse")

    def objective(H):                                    # H [npos, 4]: channel weights of every position
        n = X.size - m + 1
        act = np.zeros((X.size, nf))
        for j in range(m):
            act[:n] += H[j:j + n] @ p["Wscan"][4 * j:4 * j + 4]
        act = np.maximum(act + p["bscan"], 0)
        pooled = np.stack([act[a:b].max(axis=0) for a, b in R])
        out = pooled @ p["W1"] + p["b1"]
        return 0.5 * float((out ** 2).sum()), out
    H0 = np.where(X[:, None] == 255, 0.25, (X[:, None] == np.arange(4)).astype(float))
    _, out0 = objective(H0)
    assert np.allclose(out0, Z, rtol=1e-12, atol=1e-12)
    eps = 1e-6
    fd = np.zeros_like(H0)
    for i in range(X.size):
        for k in range(4):
            Hp, Hm = H0.copy(), H0.copy()
            Hp[i, k] += eps; Hm[i, k] -= eps
            fd[i, k] = (objective(Hp)[0] - objective(Hm)[0]) / (2 * eps)
    assert np.abs(dX).max() > 0
    assert np.max(np.abs(fd - dX)) <= 1e-6 * np.abs(dX).max() + 1e-8
