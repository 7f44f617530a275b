"""The ordinal encoding and the reverse complement against the reference's own code: the
fixture tests/golden/ref_util_tables.npz holds what kangaroo/util.py:40-116 (executed as it
stands by tests/golden/make_ref_util.py) computes -- its three 256-entry translation tables
and its revcomp / acgtcomplement of sample strings with every kind of byte."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ref():
    d = np.load(os.path.join(HERE, "golden", "ref_util_tables.npz"))
    split = lambda a: bytes(a).decode("latin-1").split("\n")
    return {"acgt2ord": d["acgt2ord"], "complement": d["complement"], "ord2acgt": d["ord2acgt"],
            "texts": split(d["texts"]), "revcomps": split(d["revcomps"]), "complements": split(d["complements"])}


def test_oracle_encoding_equals_the_reference_table(ref):
    from oracle import oracle as orc
    every = bytes(range(256)).decode("latin-1")
    np.testing.assert_array_equal(orc.acgt2ord(every), ref["acgt2ord"])
    assert set(np.unique(ref["acgt2ord"])) == {0, 1, 2, 3, 255}


def test_oracle_reverse_complement_equals_the_reference(ref):
    from oracle import oracle as orc
    assert len(ref["texts"]) == len(ref["revcomps"]) == 45
    for t, want, comp in zip(ref["texts"], ref["revcomps"], ref["complements"]):
        assert orc.revcomp(t) == want
        assert want == comp[::-1]
        # the complement table applied byte by byte is what the reference's translate() did
        assert bytes(ref["complement"][np.frombuffer(t.encode("latin-1"), np.uint8)]).decode("latin-1") == comp


def test_ordinal_reverse_complement_commutes_with_the_encoding(ref):
    """synth.revcomp_ord works on ordinals; the reference works on text and encodes afterwards."""
    from deepbind_b200 import synth
    enc = lambda s: ref["acgt2ord"][np.frombuffer(s.encode("latin-1"), np.uint8)]
    for t, rc in zip(ref["texts"], ref["revcomps"]):
        np.testing.assert_array_equal(synth.revcomp_ord(enc(t)), enc(rc))


@pytest.mark.gpu
@pytest.mark.parametrize("pad", [0, 15, 23])
def test_device_batch_builder_equals_the_reference_encoding(cuda, ref, pad):
    """db_build_batch on the sample strings, both strands: every forward row is the reference's
    table applied to the text, every reverse-complement row the table applied to the reference's
    revcomp of it; pads are 255 (kangaroo/data.py:329-334)."""
    from deepbind_b200 import fused
    texts = ref["texts"]
    X, R = fused.build_batch(texts, pad, True, device=cuda)
    X, R = X.cpu().numpy(), R.cpu().numpy()
    enc = lambda s: ref["acgt2ord"][np.frombuffer(s.encode("latin-1"), np.uint8)]
    assert R.shape == (2 * len(texts), 2)
    covered = np.zeros(X.size, bool)
    for i, (t, rc) in enumerate(zip(texts, ref["revcomps"])):
        for row, s in ((2 * i, t), (2 * i + 1, rc)):
            r0, r1 = int(R[row, 0]), int(R[row, 1])
            assert r1 - r0 == pad + len(s)
            np.testing.assert_array_equal(X[r0 + pad:r1], enc(s))
            covered[r0 + pad:r1] = True
    assert (X[~covered] == 255).all() and X.size == int(R[-1, 1]) + pad


def _batches():
    d = np.load(os.path.join(HERE, "golden", "ref_util_tables.npz"))
    k = 0
    while "b%d_X" % k in d.files:
        seqs = bytes(d["b%d_seqs" % k]).decode("latin-1").split("\n")
        padding, rc = (int(v) for v in d["b%d_padding_rc" % k])
        yield seqs, padding, bool(rc), d["b%d_X" % k], d["b%d_R" % k]
        k += 1


def test_oracle_batch_assembly_equals_the_reference_statements():
    """oracle.asbatch against the ordinal buffer and region table that the reference's own
    batch-assembly statements (kangaroo/data.py:283-284,326-334) produced."""
    from oracle import oracle as orc
    n = 0
    for seqs, padding, rc, X, R in _batches():
        gotX, gotR = orc.asbatch(seqs, padding, reverse_complement=rc)
        np.testing.assert_array_equal(gotX, X)
        np.testing.assert_array_equal(gotR, R)
        n += 1
    assert n == 4


def test_host_packing_equals_the_reference_statements():
    """synth.pack_batch (the host-side packer of ordinal arrays) gives the same layout."""
    from deepbind_b200 import synth
    from oracle import oracle as orc
    for seqs, padding, rc, X, R in _batches():
        if rc:
            continue
        gotX, gotR = synth.pack_batch([orc.acgt2ord(s) for s in seqs], padding + 1)
        np.testing.assert_array_equal(gotX, X)
        np.testing.assert_array_equal(gotR, R)


@pytest.mark.gpu
def test_device_batch_builder_equals_the_reference_statements(cuda):
    from deepbind_b200 import fused
    for seqs, padding, rc, X, R in _batches():
        gotX, gotR = fused.build_batch(seqs, padding, rc, device=cuda)
        np.testing.assert_array_equal(gotX.cpu().numpy(), X)
        np.testing.assert_array_equal(gotR.cpu().numpy().view(np.uint32), R)


def test_oracle_strand_selection_equals_the_reference_function():
    """The stronger strand of each forward / reverse-complement pair, the forward one on ties,
    against what the reference's maskout_revcomp (kangaroo/predict.py:144-164) kept."""
    from oracle import oracle as orc
    d = np.load(os.path.join(HERE, "golden", "ref_util_tables.npz"))
    Z, kept, mask = d["strand_Z"], d["strand_kept"], d["strand_mask"]
    assert kept.shape == (32, 1) and mask.sum() == 32
    np.testing.assert_array_equal(orc.strand_max_rows(Z), kept)
    pairs = Z.reshape(-1, 2)
    np.testing.assert_array_equal(mask.reshape(-1, 2)[:, 0], pairs[:, 0] >= pairs[:, 1])


@pytest.mark.gpu
def test_device_strand_selection_equals_the_reference_function(cuda):
    import torch
    from deepbind_b200 import _lib
    d = np.load(os.path.join(HERE, "golden", "ref_util_tables.npz"))
    Z = torch.from_numpy(d["strand_Z"]).to(cuda)
    out = torch.empty((32, 1), dtype=torch.float32, device=cuda)
    _lib.load().db_strand_max(out.data_ptr(), Z.data_ptr(), 32, 1)
    got = out.cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), d["strand_kept"].view(np.uint32))     # the kept row's own bits, signed zeros included
