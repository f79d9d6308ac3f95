"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations.  They stand in for CMS HGCAL events (which are not distributable): uniform
points, Gaussian "showers" on uniform noise, and Gaussian blobs with a beta spectrum.

Everything is generated with ``numpy.random.default_rng(seed)`` and cast to float32 / int32, so
the CPU checker and the CUDA library always see identical arrays.
"""
from __future__ import annotations

import numpy as np


def uniform_event(n_hits=20000, dims=3, n_feat=32, seed=101):
    """One event of uniform hits in [0,1)^dims with N(0,1) features."""
    rng = np.random.default_rng(seed)
    coords = rng.random((n_hits, dims), dtype=np.float32)
    feats = rng.standard_normal((n_hits, n_feat), dtype=np.float32)
    row_splits = np.array([0, n_hits], np.int32)
    return coords, feats, row_splits


def shower_event(n_hits, dims=4, n_showers=300, noise_fraction=0.1, seed=200):
    """Coordinates of one event: isotropic Gaussian showers (centres U[-1,1]^dims, sigma
    U(0.01,0.05), exponentially distributed sizes) plus uniform noise in [-1,1]^dims, shuffled."""
    rng = np.random.default_rng(seed)
    n_noise = int(round(noise_fraction * n_hits))
    n_sig = n_hits - n_noise
    centres = rng.uniform(-1., 1., (n_showers, dims))
    sigma = rng.uniform(0.01, 0.05, n_showers)
    w = rng.exponential(1., n_showers)
    counts = np.floor(n_sig * w / w.sum()).astype(np.int64)
    counts[0] += n_sig - counts.sum()
    label = np.repeat(np.arange(n_showers), counts)
    sig = centres[label] + sigma[label, None] * rng.standard_normal((n_sig, dims))
    noise = rng.uniform(-1., 1., (n_noise, dims))
    coords = np.concatenate([sig, noise], axis=0)
    rng.shuffle(coords, axis=0)
    return coords.astype(np.float32)


def shower_batch(event_sizes, dims=4, n_feat=64, seed=200, with_features=True):
    """A ragged batch of shower events; event e uses seed ``seed + e``."""
    coords = [shower_event(int(n), dims=dims, seed=seed + e) for e, n in enumerate(event_sizes)]
    row_splits = np.concatenate([[0], np.cumsum(event_sizes)]).astype(np.int32)
    coords = np.concatenate(coords, axis=0)
    feats = None
    if with_features:
        rng = np.random.default_rng(seed + 100000)
        feats = rng.standard_normal((coords.shape[0], n_feat), dtype=np.float32)
    return coords, feats, row_splits


def ragged_shower_batch(n_events=4, lo=50000, hi=150000, dims=4, n_feat=64, seed=200):
    """Event sizes drawn uniformly in [lo, hi]."""
    sizes = np.random.default_rng(seed - 1).integers(lo, hi + 1, n_events)
    return shower_batch(sizes, dims=dims, n_feat=n_feat, seed=seed)


def condensation_batch(n_events=4, n_hits=200000, n_blobs=500, dims=3, sigma=0.1, seed=400):
    """Cluster coordinates as Gaussian blobs (centres U[-3,3]^dims), beta ~ Beta(0.5,5) with the
    hit closest to each blob centre promoted to beta ~ U(0.8,1)."""
    cc, bb = [], []
    for e in range(n_events):
        rng = np.random.default_rng(seed + e)
        centres = rng.uniform(-3., 3., (n_blobs, dims))
        label = rng.integers(0, n_blobs, n_hits)
        x = centres[label] + sigma * rng.standard_normal((n_hits, dims))
        beta = rng.beta(0.5, 5., n_hits)
        d2 = ((x - centres[label]) ** 2).sum(axis=1)
        order = np.lexsort((d2, label))
        first = np.concatenate([[True], label[order][1:] != label[order][:-1]])
        seeds = order[first]
        beta[seeds] = rng.uniform(0.8, 1., len(seeds))
        cc.append(x.astype(np.float32))
        bb.append(beta.astype(np.float32))
    row_splits = (np.arange(n_events + 1) * n_hits).astype(np.int32)
    return np.concatenate(cc), np.concatenate(bb)[:, None], row_splits


def gravnet_weights(block, f_in=64, coord_dims=4, f_out=64):
    """Random-initialised dense weights of one GravNet-style block (fixed seeds)."""
    wc = np.random.default_rng(310 + block).normal(0., np.sqrt(1. / f_in), (f_in, coord_dims))
    wo = np.random.default_rng(320 + block).normal(0., np.sqrt(1. / (3 * f_in)), (3 * f_in, f_out))
    return wc.astype(np.float32), wo.astype(np.float32)
