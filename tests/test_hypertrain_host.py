"""Host-side bookkeeping of calibration: folds, metrics, best-sample choice (no GPU)."""
import numpy as np


def test_split_folds_follow_datasource_split():
    from deepbind_b200.hypertrain import split_folds
    A, B = split_folds(10, 0, 1)
    assert A.tolist() == [0, 1, 2, 3, 4] and B.tolist() == [5, 6, 7, 8, 9]
    A, B = split_folds(10, 1, 1)
    assert A.tolist() == [5, 6, 7, 8, 9] and B.tolist() == [0, 1, 2, 3, 4]
    # nsplit = 3: blocks at linspace(0, 10, 5) = 0, 2, 5, 7, 10; index 1 holds out block 2
    A, B = split_folds(10, 1, 3)
    assert B.tolist() == [5, 6] and A.tolist() == [0, 1, 2, 3, 4, 7, 8, 9]
    # every row is held out exactly once over the k folds
    held = np.concatenate([split_folds(20000, f, 2)[1] for f in range(3)])
    assert sorted(held.tolist()) == list(range(20000))
    A, B = split_folds(7, 0, 0)
    assert A.tolist() == list(range(7)) and B.size == 0


def test_auc_and_pearson():
    from sklearn.metrics import roc_auc_score
    from scipy.stats import pearsonr
    from deepbind_b200.hypertrain import calc_auc, pearson
    rng = np.random.default_rng(0)
    y = rng.integers(0, 2, 500).astype(np.float32)
    z = rng.standard_normal(500) + y            # informative, no ties
    assert abs(calc_auc(z, y) - roc_auc_score(y, z)) < 1e-12
    assert calc_auc(y, y) == 1.0 and np.isnan(calc_auc(z, np.ones(500)))
    assert abs(pearson(z, y) - pearsonr(z, y)[0]) < 1e-12
    assert np.isnan(pearson(np.ones(5), np.arange(5)))


def test_best_sample_skips_nan_and_keeps_the_first_best():
    from deepbind_b200.hypertrain import get_best_sample
    recs = [{"value": float("nan"), "id": 0}, {"value": 0.7, "id": 1}, {"value": 0.9, "id": 2}, {"value": 0.9, "id": 3}]
    assert get_best_sample(recs, wantmax=True)["id"] == 2
    assert get_best_sample(recs, wantmax=False)["id"] == 1
    assert get_best_sample([{"value": float("nan")}]) is None
