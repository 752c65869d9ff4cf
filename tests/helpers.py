"""Shared helpers for the tests: packed-metadata decoding and oracle conveniences."""
import math

import numpy as np
import torch

from oracle import tree_oracle as orc


def packed_offsets(nb, bm, ma):
    """Byte offsets of count / idx / mask / leaf inside one packed blob (16-byte aligned parts)."""
    a16 = lambda x: (x + 15) & ~15
    maw, lw = (ma + 31) // 32, (bm + 31) // 32
    off_idx = a16(nb * 4)
    off_mask = off_idx + a16(nb * ma * 4)
    off_leaf = off_mask + a16(nb * bm * maw * 4)
    total = off_leaf + a16(nb * lw * 4)
    return off_idx, off_mask, off_leaf, total, maw, lw


def decode_packed(blob: np.ndarray, nb, bm, ma):
    """Packed blob (uint8 array) -> reference-format arrays (int64 idx, bool mask, int64 leaf)."""
    off_idx, off_mask, off_leaf, total, maw, lw = packed_offsets(nb, bm, ma)
    assert blob.shape[0] >= total
    count = blob[: nb * 4].view(np.int32)
    idx = blob[off_idx: off_idx + nb * ma * 4].view(np.int32).reshape(nb, ma)
    words = blob[off_mask: off_mask + nb * bm * maw * 4].view(np.uint32).reshape(nb, bm, maw)
    bits = np.unpackbits(words.view(np.uint8).reshape(nb, bm, maw * 4), axis=2, bitorder="little")
    mask = bits[:, :, :ma].astype(bool)
    leafw = blob[off_leaf: off_leaf + nb * lw * 4].view(np.uint32).reshape(nb, lw)
    leafbits = np.unpackbits(leafw.view(np.uint8).reshape(nb, lw * 4), axis=1, bitorder="little")[:, :bm]
    rows = np.arange(nb)[:, None] * bm + np.arange(bm)[None, :]
    leaf = np.where(leafbits.astype(bool), rows, -1).astype(np.int64)
    return count.copy(), idx.astype(np.int64), mask, leaf


def chain_mean_values(parent, v):
    """With all-equal scores every node averages V over itself and its ancestors.

    v: [..., N, D] float64 array -> same shape; computed by a running sum down the tree.
    """
    n = len(parent)
    s = np.array(v, dtype=np.float64, copy=True)
    depth = np.zeros(n)
    for i in range(n):
        p = parent[i]
        if p >= 0:
            s[..., i, :] += s[..., p, :]
            depth[i] = depth[p] + 1
    return s / (depth + 1)[:, None]


def make_qkv(z, h, n_q, n_kv, d, dtype, seed, device="cuda", std=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((z, h, n_q, d), generator=g) * std).to(dtype)
    k = (torch.randn((z, h, n_kv, d), generator=g) * std).to(dtype)
    v = (torch.randn((z, h, n_kv, d), generator=g) * std).to(dtype)
    return q, k, v


def oracle_attention(q, k, v, parent, sm_scale, prefix=0, compute_dtype=None, head_chunk=None):
    """Dense oracle on CPU tensors whose q has exactly len(parent) rows (no padding needed)."""
    lin, _ = orc.lineage_from_parent(parent)
    mask = orc.full_attention_mask(lin, pad_rows=0)
    if prefix:
        mask = torch.cat((torch.ones((mask.shape[0], prefix)), mask), dim=1)
    return orc.dense_tree_attention(q, k, v, mask, sm_scale, compute_dtype, head_chunk)


def pad_rows(n, bm):
    return math.ceil(n / bm) * bm
