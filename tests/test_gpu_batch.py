"""Device-side minibatch assembly against the oracle's restatement of kangaroo's
packing (data.py:274-334, util.py:43-74): byte for byte, index for index."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ALPHABET = np.frombuffer(b"ACGTUNacgtunRYxz.-*", dtype=np.uint8)


def random_seqs(rng, nseq, lmin, lmax, alphabet=ALPHABET):
    return [alphabet[rng.integers(0, alphabet.size, rng.integers(lmin, lmax + 1))].tobytes().decode("latin-1") for _ in range(nseq)]


@pytest.mark.parametrize("rc", [False, True])
@pytest.mark.parametrize("nseq,lmin,lmax,pad", [(1, 1, 1, 0), (1, 40, 40, 23), (37, 0, 90, 15), (500, 20, 200, 23),
                                               (3000, 101, 101, 23), (64, 0, 0, 4), (9, 1, 700, 1)])
def test_batch_equals_oracle(cuda, orc, nseq, lmin, lmax, pad, rc):
    from deepbind_b200 import fused
    rng = np.random.default_rng(nseq * 31 + pad + rc)
    seqs = random_seqs(rng, nseq, lmin, lmax)
    wantX, wantR = orc.asbatch(seqs, pad, rc)
    X, R = fused.build_batch(seqs, pad, rc)
    assert np.array_equal(X.cpu().numpy(), wantX)
    assert np.array_equal(R.cpu().numpy().view(np.uint32), wantR)


def test_empty_batch_is_one_pad(cuda, orc):
    from deepbind_b200 import fused
    X, R = fused.build_batch([], 7)
    wantX, _ = orc.asbatch([], 7)
    assert np.array_equal(X.cpu().numpy(), wantX) and R.shape == (0, 2)


def test_device_text_with_nonzero_first_offset(cuda, orc):
    """A window of a larger device-resident text: offsets[0] != 0."""
    import torch
    from deepbind_b200 import fused
    rng = np.random.default_rng(5)
    seqs = random_seqs(rng, 50, 10, 60)
    raw = "".join(seqs).encode("latin-1")
    off = np.concatenate([[0], np.cumsum([len(s) for s in seqs])]).astype(np.int32)
    text = torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()
    X, R = fused.build_batch((text, torch.from_numpy(off[10:31].copy()).cuda()), 12, True)
    wantX, wantR = orc.asbatch(seqs[10:30], 12, True)
    assert np.array_equal(X.cpu().numpy(), wantX)
    assert np.array_equal(R.cpu().numpy().view(np.uint32), wantR)


def test_built_batch_scores_like_the_host_built_one(cuda, orc):
    """Text -> device batch -> fused scan, both strands, equals the oracle end to end."""
    import torch
    from deepbind_b200 import fused
    rng = np.random.default_rng(8)
    m, nf = 24, 16
    seqs = random_seqs(rng, 200, 30, 120, np.frombuffer(b"ACGTN", dtype=np.uint8))
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(np.float32)
    b = rng.uniform(-0.1, 0, nf).astype(np.float32)
    X, R = fused.build_batch(seqs, m - 1, True)
    got, _, _ = fused.scanpool(torch.from_numpy(W).cuda(), torch.from_numpy(b).cuda(), X, R, "all")
    hX, hR = orc.asbatch(seqs, m - 1, True)
    want, _ = orc.scanpool(W, b, True, hX, hR, "all")
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("rc", [False, True])
@pytest.mark.parametrize("nseq,lmin,lmax,W,stride,pad", [(1, 30, 30, 20, 1, 23), (12, 1, 90, 20, 1, 15), (40, 5, 300, 33, 7, 23),
                                                        (7, 0, 10, 20, 3, 23), (5, 50, 60, 1, 1, 4), (9, 10, 40, 64, 64, 0)])
def test_windows_equal_oracle(cuda, orc, nseq, lmin, lmax, W, stride, pad, rc):
    """Scan-mode window expansion: byte for byte the batch the reference's string slicing gives."""
    from deepbind_b200 import fused
    rng = np.random.default_rng(nseq * 7 + W + stride + rc)
    seqs = random_seqs(rng, nseq, max(lmin, 1 if W == 1 else 0), lmax)
    windows = [w for s in seqs for w in orc.scan_windows(s, W, stride)]
    wantX, wantR = orc.asbatch(windows, pad, rc)
    X, R, woff = fused.build_windows(seqs, W, stride, pad, rc)
    assert woff.tolist() == np.concatenate([[0], np.cumsum([len(orc.scan_windows(s, W, stride)) for s in seqs])]).tolist()
    assert np.array_equal(X.cpu().numpy(), wantX)
    assert np.array_equal(R.cpu().numpy().view(np.uint32), wantR)
