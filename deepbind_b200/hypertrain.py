"""Calibration (hyper-parameter search with k-fold validation) and final training,
following the reference's calibrate -> train workflow
(code/libs/deepity/deepity/hypertrain.py:248-400,560-580, hpsearch.py:95-260,
kangaroo/train.py:74-172) around the device-side trainer.

* ``ncalib`` hyper-parameter samples are trained side by side as the instances of
  one :class:`DeepBindNet` (the reference's instance batching), once per fold;
* the data are shuffled once with a fixed seed, and fold ``f`` of ``nfold`` holds
  out the block ``split_folds`` describes (deepity/data.py:120-145);
* every checkpoint of every sample is scored on the held-out block; the best
  (sample, step) by validation metric gives the hyper-parameters, including the
  number of steps, of the final training (hpsearch.py:224-241);
* the final training runs ``ntrial`` differently initialised instances with those
  hyper-parameters on all the data and keeps the one that fits the training data best.

The bookkeeping is host code; every model evaluation runs through the same
kernels as training and scoring.

Several GPUs (one process per GPU, ``group`` = a torch.distributed process group, or
the default group with ``group="world"``): the hyper-parameter samples -- and the
trials of the final training -- are dealt to the ranks round robin, as the reference
hands them to one worker process per device (hpsearch.py:316-330,376); every rank
trains its own instances on the full data with no gradient exchange, and only the
validation records (host objects) and the winning trial's parameters are exchanged.
"""
import json
import os

import numpy as np

from . import cfg, shard
from .trainer import Trainer


def _group(group):
    """``"world"`` -> the default process group (None for torch.distributed calls)."""
    return None if (isinstance(group, str) and group == "world") else group


def _rank_world(group):
    if group is None:
        return 0, 1
    return shard.rank_world(_group(group))


# --------------------------------------------------------------------- metrics
def calc_auc(z, y):
    """Area under the ROC curve as deepity/report.py:56-106 computes it: stable sort
    by decreasing score, cumulative true/false positives, trapezoidal rule; NaN if
    a class is empty."""
    z = np.asarray(z, np.float64).ravel(); y = np.asarray(y, np.float64).ravel()
    assert len(z) == len(y)
    order = np.argsort(z, kind="mergesort")[::-1]
    y = y[order]
    tpr = y.cumsum()
    fpr = 1 + np.arange(len(y), dtype=np.float64) - tpr
    if fpr[0] != 0:
        tpr = np.r_[0, tpr]; fpr = np.r_[0, fpr]
    if fpr[-1] == 0 or tpr[-1] == 0:
        return np.nan
    tpr = tpr / tpr[-1]; fpr = fpr / fpr[-1]
    return float(np.sum((fpr[1:] - fpr[:-1]) * (tpr[1:] + tpr[:-1]) * 0.5))


def pearson(z, y):
    z = np.asarray(z, np.float64).ravel(); y = np.asarray(y, np.float64).ravel()
    zc, yc = z - z.mean(), y - y.mean()
    d = np.sqrt((zc * zc).sum() * (yc * yc).sum())
    return float((zc * yc).sum() / d) if d > 0 else np.nan


def split_folds(n, index=0, nsplit=1):
    """(A, B) index arrays of ``datasource.split(index, nsplit)`` (deepity/data.py:120-145):
    B is block nsplit - index of nsplit + 1 near-equal blocks, A is the rest."""
    assert index <= nsplit
    if nsplit <= 0:
        return np.arange(n), np.arange(0)
    at = [int(x) for x in np.linspace(0, n, nsplit + 2)]
    r = nsplit - index
    return np.r_[np.arange(at[0], at[r]), np.arange(at[r + 1], at[-1])], np.arange(at[r], at[r + 1])


# ----------------------------------------------------------------- calibration
def _metric_of(net, loss):
    return ("auc", True) if loss == "nll" else ("pearson", True)


def _validate(net, seqs, Y, batch=4096):
    """Scores of every instance on held-out sequences, in test mode -> (Z [n, I])."""
    from .predict import predict
    out = []
    for lo in range(0, len(seqs), batch):
        out.append(predict(net, seqs[lo:lo + batch])["direct"].cpu().numpy())
    return np.concatenate(out) if out else np.zeros((0, net.I), np.float32)


def calibrate(layers, trainer_spec, seqs, Y, ncalib=30, nfold=3, seed=0, motif_len=None, shuffle_seed=1234, outdir=None,
              allfolds=True, group=None):
    """Draws ``ncalib`` hyper-parameter samples, trains each on every fold, validates
    every checkpoint.  Returns a list of records
    ``{"sample", "step", "hparams", "metric", "value", "folds"}`` (one per sample and
    checkpoint; ``value`` is the mean of the folds' validation metric) and the best
    record.  With ``outdir`` the records are also written to ``calib.all.json``
    (by rank 0).  With ``group`` the samples are dealt to the group's ranks; every rank
    returns the records of all samples."""
    rank, world = _rank_world(group)
    mine = shard.shard_models(ncalib, rank, world)          # this rank's samples
    seqs = list(seqs)
    Y = np.asarray(Y, np.float32).reshape(len(seqs), -1)
    perm = np.random.default_rng(shuffle_seed).permutation(len(seqs))       # always the same shuffle, hence the same folds
    seqs = [seqs[i] for i in perm]; Y = Y[perm]
    records = {}
    metric = None
    for fold in range(nfold if allfolds else 1):
        A, B = split_folds(len(seqs), fold, nfold - 1)
        # the same draws for every fold: a sample is a hyper-parameter set, evaluated nfold times
        # (a rank left without a sample still draws, for the record of hyper-parameters)
        keep = (mine or [0]) if world > 1 else None
        net, drawn = cfg.instantiate(layers, ninst=ncalib, seed=seed, motif_len=motif_len, instances=keep)
        tr = Trainer(net, trainer_spec, seed=seed, ninst=ncalib, instances=keep)
        metric, _ = _metric_of(net, net.loss)
        vseqs, vY = ([seqs[i] for i in B], Y[B]) if len(B) else ([seqs[i] for i in A], Y[A])

        def on_checkpoint(step, trainer):
            Z = _validate(trainer.net, vseqs, vY)
            for col, s in enumerate(mine):
                v = calc_auc(Z[:, col], vY[:, 0]) if metric == "auc" else pearson(Z[:, col], vY[:, 0])
                rec = records.setdefault((s, step), {"sample": s, "step": step, "metric": metric, "folds": []})
                rec["folds"].append(v)
        if mine:
            tr.fit([seqs[i] for i in A], Y[A], on_checkpoint=on_checkpoint)
        hp = {k: np.asarray(v).tolist() for k, v in drawn.items()}
        hp["trainer.rate"], hp["trainer.momentum"] = tr.rate_all.tolist(), tr.momentum_all.tolist()
    if world > 1:                                            # every rank learns every sample's records
        records = {k: v for part in shard.gather_objects(records, _group(group)) for k, v in part.items()}
    out = []
    for (s, step), rec in sorted(records.items()):
        rec["hparams"] = {k: v[s] for k, v in hp.items()}
        rec["value"] = float(np.mean(rec["folds"])) if not np.any(np.isnan(rec["folds"])) else float("nan")
        out.append(rec)
    best = get_best_sample(out, wantmax=True)
    if outdir and rank == 0:
        os.makedirs(outdir, exist_ok=True)
        with open(os.path.join(outdir, "calib.all.json"), "w") as f:
            json.dump({"records": out, "best": best}, f, indent=1)
    return out, best


def get_best_sample(records, wantmax=False):
    """hpsearch.py:224-241: the first record with the best non-NaN value."""
    best = None
    for r in records:
        if not np.isnan(r["value"]):
            if best is None or (r["value"] > best["value"] if wantmax else r["value"] < best["value"]):
                best = r
    return best


def _fix(layers, hparams, ntrial):
    """The layer list with every drawn range replaced by the chosen value, once per trial."""
    import copy
    fixed_layers = copy.deepcopy(layers)
    for key, val in hparams.items():
        if key.startswith("trainer."):
            continue
        idx, _, arg = key.split(".")
        setattr(fixed_layers[int(idx)], arg, cfg.fixed(np.full(ntrial, val)))
    return fixed_layers


def train_final(layers, trainer_spec, best, seqs, Y, ntrial=3, seed=0, motif_len=None, group=None):
    """Trains ``ntrial`` instances with the best record's hyper-parameters and step
    count on all the data; returns (net, index of the trial with the best training
    metric, metrics [ntrial]).  With ``group`` the trials are dealt to the ranks
    (a rank without a trial idles); the returned net then holds this rank's trials
    only (None on a rank without any), ``metrics`` all trials', and
    :func:`best_trial_params` hands the winner's parameters to every rank."""
    import copy
    rank, world = _rank_world(group)
    mine = shard.shard_models(ntrial, rank, world)
    spec = copy.copy(trainer_spec)
    spec.rate, spec.momentum = best["hparams"]["trainer.rate"], best["hparams"]["trainer.momentum"]
    spec.max_steps, spec.checkpoints = int(best["step"]), 1
    Yv = np.asarray(Y, np.float32).reshape(len(seqs), -1)
    net, local = None, []
    if mine:
        net, _ = cfg.instantiate(_fix(layers, best["hparams"], ntrial), ninst=ntrial, seed=seed + 1, motif_len=motif_len,
                                 instances=mine if world > 1 else None)
        Trainer(net, spec, seed=seed, ninst=ntrial, instances=mine if world > 1 else None).fit(list(seqs), Y)
        Z = _validate(net, list(seqs), Yv)
        local = [calc_auc(Z[:, c], Yv[:, 0]) if net.loss == "nll" else pearson(Z[:, c], Yv[:, 0]) for c in range(len(mine))]
    vals = np.asarray(shard.deal_back(shard.gather_objects(local, _group(group)), ntrial, world) if world > 1 else local)
    return net, int(np.nanargmax(vals)), vals


def best_trial_params(net, best_trial, ntrial, group=None):
    """The parameter blocks (numpy, one instance) of trial ``best_trial`` of a final
    training whose ``ntrial`` trials were dealt to the ranks of ``group``: the owning
    rank cuts them out of its net, every rank receives them."""
    rank, world = _rank_world(group)
    owner = best_trial % world
    params = None
    if rank == owner:
        col = shard.shard_models(ntrial, rank, world).index(best_trial) if world > 1 else best_trial
        params = cfg.select_instances(net.params_numpy("P"), np.asarray([col]), net.I)
    if world > 1:
        import torch.distributed as dist
        box = [params]
        dist.broadcast_object_list(box, src=dist.get_global_rank(_group(group), owner) if _group(group) is not None else owner,
                                   group=_group(group))
        params = box[0]
    return params


# ------------------------------------------------------------------ persistence
def save_model(path, net, instance=None, meta=None):
    """Writes the trained model to ``path`` (.npz): the parameter blocks, and what is
    needed to rebuild the net (pooling, loss, dropout rates, number of instances) plus
    ``meta`` (any JSON-serialisable record, e.g. the chosen hyper-parameters) -- the
    counterpart of the reference's ``model.pkl`` (kangaroo/train.py:150-172).
    ``instance``: keep only that instance (e.g. the best trial of ``train_final``)."""
    P = net.params_numpy("P")
    I = net.I
    rate = None if net.dropout_rate is None else np.asarray(net.dropout_rate, np.float32)
    if instance is not None:
        t, out = int(instance), {}
        for k, w in P.items():
            if k in ("W1", "W2"):                 # instances stacked on rows
                rows = w.shape[0] // I
                out[k] = w[t * rows:(t + 1) * rows]
            else:                                 # instances side by side on columns
                cols = w.shape[-1] // I
                out[k] = w[..., t * cols:(t + 1) * cols]
        P, I = out, 1
        rate = None if rate is None else rate[t:t + 1]
    info = {"nmodel": I, "pool": net.pool, "loss": net.loss, "dropout_rate": None if rate is None else rate.tolist(),
            "meta": meta}
    np.savez(path, __info__=np.frombuffer(json.dumps(info).encode(), np.uint8), **P)


def load_model(path, device=None):
    """Rebuilds the net written by ``save_model``; returns (net, meta)."""
    from .model import DeepBindNet
    with np.load(path) as f:
        info = json.loads(bytes(f["__info__"]).decode())
        P = {k: f[k] for k in f.files if k != "__info__"}
    net = DeepBindNet(P, info["nmodel"], info["pool"], loss=info["loss"], device=device)
    if info["dropout_rate"] is not None:
        net.set_dropout(np.asarray(info["dropout_rate"], np.float32))
    return net, info["meta"]
