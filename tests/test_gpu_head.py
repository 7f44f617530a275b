"""The one-launch dense head (db_head_train) against the operator-by-operator head
and against the CPU oracle: loss and every gradient within 1e-5 of the largest
gradient entry (the two paths sum in different orders)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)).cuda()


@pytest.mark.parametrize("I,pool,hidden,loss,B,use_mask", [(1, "all", 32, "nll", 128, True), (7, "max", 0, "mse", 64, False),
                                                           (3, "all", 8, "mse", 37, True), (90, "max", 0, "mse", 64, False)])
def test_fused_head_matches_unfused_and_oracle(cuda, orc, I, pool, hidden, loss, B, use_mask):
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m = 24
    p = synth.model_params(I, m, 13, pool, hidden=hidden)
    X, R = synth.ragged_batch(B, 30, 80, m, seed=14, n_frac=0.02)
    g = synth.rng(15)
    Y = np.tile((g.integers(0, 2, size=(B, 1)) if loss == "nll" else g.standard_normal((B, 1))).astype(np.float32), (1, I))
    npool = 16 * (2 if pool == "all" else 1)
    mask = (g.random((B, npool * I)) >= 0.5) if use_mask else None
    tX, tR, tY = dev(X), dev(R), dev(Y)
    tM = dev(mask) if use_mask else None
    a = DeepBindNet(p, I, pool, loss=loss, fused_head=True)
    b = DeepBindNet(p, I, pool, loss=loss, fused_head=False)
    La = a.grads(tX, tR, tY, tM).cpu().numpy()
    Lb = b.grads(tX, tR, tY, tM).cpu().numpy()
    Lw, gw = orc.train_grads(p, X, R, Y, pool, I, loss, mask)
    np.testing.assert_allclose(La, Lw, rtol=1e-5)
    np.testing.assert_allclose(Lb, Lw, rtol=1e-5)
    ga, gb = a.params_numpy("dP"), b.params_numpy("dP")
    for k, w in gw.items():
        scale = max(np.abs(w).max(), 1e-6)
        assert np.max(np.abs(ga[k].reshape(w.shape) - w)) <= 1e-5 * scale, k
        assert np.max(np.abs(gb[k].reshape(w.shape) - w)) <= 1e-5 * scale, k


def test_minibatch_beyond_the_tile_uses_the_operator_path(cuda):
    import torch
    from deepbind_b200 import _lib, synth, SmatException
    from deepbind_b200.model import DeepBindNet
    dll = _lib.load()
    cap = dll.db_head_max_batch(32, 32)
    assert 128 <= cap < 4096
    z = torch.zeros(8, device="cuda")
    with pytest.raises(SmatException, match="exceeds the fused head"):
        dll.db_head_train(1, 32, 32, 1, 0, cap + 64, z.data_ptr(), None, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                          z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr())
    # DeepBindNet falls back to separate operators for such a batch and still trains
    B = cap + 64
    p = synth.model_params(1, 24, 1, "all", hidden=32)
    X, R = synth.uniform_batch(B, 30, 24, seed=2)
    net = DeepBindNet(p, 1, "all")
    L = net.grads(dev(X), dev(R), dev(np.zeros((B, 1), np.float32)))
    assert np.isfinite(L.cpu().numpy()).all()


@pytest.mark.parametrize("fused_head", [True, False])
@pytest.mark.parametrize("I,pool,hidden,loss", [(1, "max", 0, "mse"), (3, "all", 32, "nll")])
def test_two_strand_training_masks_the_weaker_strand(cuda, orc, I, pool, hidden, loss, fused_head):
    """Rows are forward / reverse-complement pairs: only the stronger row of each pair carries
    loss and gradient (calc_zmask + maskout, loss.py:52-65,98-117), the mean divides by all rows."""
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, nseq = 24, 48
    p = synth.model_params(I, m, 21, pool, hidden=hidden)
    X, R = synth.ragged_batch(nseq, 30, 80, m, seed=22, n_frac=0.02, both_strands=True)
    g = synth.rng(23)
    y = (g.integers(0, 2, size=(nseq, 1)) if loss == "nll" else g.standard_normal((nseq, 1))).astype(np.float32)
    Y = np.tile(np.repeat(y, 2, axis=0), (1, I))                # both strands share the target
    net = DeepBindNet(p, I, pool, loss=loss, fused_head=fused_head)
    net.strand_pairs = True
    L = net.grads(dev(X), dev(R), dev(Y)).cpu().numpy()
    Lw, gw = orc.train_grads(p, X, R, Y, pool, I, loss, strand_pairs=True)
    np.testing.assert_allclose(L, Lw, rtol=1e-5)
    got = net.params_numpy("dP")
    for k, w in gw.items():
        assert np.max(np.abs(got[k].reshape(w.shape) - w)) <= 1e-5 * max(np.abs(w).max(), 1e-6), k
    # and it differs from treating the rows as independent samples
    L2, _ = orc.train_grads(p, X, R, Y, pool, I, loss)
    assert not np.allclose(Lw, L2)
