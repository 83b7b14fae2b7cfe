"""TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU oracle of the sampled-softmax head: the candidate set and the float64
cross-entropy over it. Only tests import this module.

Follows the head the reference names in include/marincpp/model.hpp:236-239 (candidates = sort-unique targets of the
device microbatch + golden-ratio stride negatives, remapped targets, gathered W_P, fused CE, unique-row scatter of dW_P)
and its gate, a float64 full-vocabulary CE whose logits are masked to the candidate set (docs/DESIGN.md:1283); the
reference ships neither code nor vectors for it, so the stride rule below is this build's reading of "golden-ratio
stride": the integer nearest V (sqrt(5) - 1) / 2, moved up to the next value coprime with V.
"""
import math

import numpy as np

import ce_oracle


def sampled_stride(V):
    if V <= 2:
        return 1
    s = int(V * 0.6180339887498949 + 0.5)
    s = max(1, min(s, V - 1))
    while math.gcd(s, V) != 1:
        s += 1
    return s


def candidates(targets, weight, V, n_negatives, neg_offset, ignore_index=None):
    """sorted unique ids: the targets of the rows that count, and n_negatives strided ids starting at neg_offset"""
    targets = np.asarray(targets).astype(np.int64)
    counts = (targets >= 0) & (targets < V) & (np.asarray(weight) != 0)
    if ignore_index is not None:
        counts &= targets != ignore_index
    first = int(neg_offset) % V
    neg = (first + np.arange(n_negatives, dtype=np.int64) * sampled_stride(V)) % V
    return np.unique(np.concatenate([targets[counts], neg])).astype(np.int32), counts


def sampled_ce_f64(x, w, targets, weight, grad_scale, n_negatives, neg_offset, z_loss=0.0, ignore_index=None):
    """Returns (loss [T], lse [T], dx [T, D], dw [V, D] (non-zero on candidate rows only), candidates)."""
    V = w.shape[0]
    cand, counts = candidates(targets, weight, V, n_negatives, neg_offset, ignore_index)
    remap = np.full(V, -1, np.int64)
    remap[cand] = np.arange(cand.size)
    t = np.asarray(targets).astype(np.int64)
    tp = np.where(counts, remap[np.clip(t, 0, V - 1)], -1)
    loss, lse, dx, dwp = ce_oracle.ce_f64(x, np.asarray(w)[cand], tp, weight, grad_scale, z_loss=z_loss)
    dw = np.zeros((V, w.shape[1]))
    dw[cand] = dwp
    return loss, lse, dx, dw, cand


def masked_full_ce_f64(x, w, targets, weight, grad_scale, cand, z_loss=0.0, ignore_index=None):
    """The gate: the full-vocabulary float64 CE with every logit outside the candidate set at -inf."""
    V = w.shape[0]
    bias = np.full(V, -np.inf)
    bias[cand] = 0.0
    return ce_oracle.ce_f64(x, w, targets, weight, grad_scale, z_loss=z_loss, ignore_index=ignore_index, bias=bias)
