"""Shared helpers for the tests: packed-metadata decoding and oracle conveniences."""
import math

import numpy as np
import torch

from oracle import tree_oracle as orc


def packed_offsets(nb, bm, ma):
    """Byte offsets of count / idx / emask / bmask inside one packed blob (16-byte aligned parts)."""
    a16 = lambda x: (x + 15) & ~15
    maw, bw = (ma + 31) // 32, (bm + 31) // 32
    off_idx = a16(nb * 4)
    off_emask = off_idx + a16(nb * ma * 4)
    off_bmask = off_emask + a16(nb * bm * maw * 4)
    total = off_bmask + a16(nb * bm * bw * 4)
    return off_idx, off_emask, off_bmask, total, maw, bw


def _bits(words, width):
    """uint32 words [..., W] -> bool [..., width] (bit i of word w is column 32 w + i)."""
    flat = np.ascontiguousarray(words).view(np.uint8).reshape(words.shape[:-1] + (words.shape[-1] * 4,))
    return np.unpackbits(flat, axis=-1, bitorder="little")[..., :width].astype(bool)


def decode_packed_raw(blob: np.ndarray, nb, bm, ma):
    """Packed blob (uint8 array) -> (count [nb], idx [nb, ma], emask [nb, bm, ma], bmask [nb, bm, bm])."""
    off_idx, off_emask, off_bmask, total, maw, bw = packed_offsets(nb, bm, ma)
    assert blob.shape[0] >= total
    count = blob[: nb * 4].view(np.int32).copy()
    idx = blob[off_idx: off_idx + nb * ma * 4].view(np.int32).reshape(nb, ma).astype(np.int64)
    emask = _bits(blob[off_emask: off_emask + nb * bm * maw * 4].view(np.uint32).reshape(nb, bm, maw), ma)
    bmask = _bits(blob[off_bmask: off_bmask + nb * bm * bw * 4].view(np.uint32).reshape(nb, bm, bw), bm)
    return count, idx, emask, bmask


def decode_packed(blob: np.ndarray, nb, bm, ma):
    """Packed blob -> the reference's three arrays (int64 idx, bool mask, int64 leaf).

    The reference's ancestor list of a block is the external list followed by the in-block
    ancestors (columns some *other* row attends to); a row is a leaf when nobody else attends
    to it.  Only exact when the full list fits in ``ma`` slots.
    """
    count, idx, emask, bmask = decode_packed_raw(blob, nb, bm, ma)
    ai = np.full((nb, ma), -1, np.int64)
    am = np.zeros((nb, bm, ma), bool)
    li = np.full((nb, bm), -1, np.int64)
    for b in range(nb):
        c = int(count[b])
        assert np.all(idx[b, c:] == -1) and not emask[b, :, c:].any()
        others = bmask[b] & ~np.eye(bm, dtype=bool)
        inblock = np.nonzero(others.any(axis=0))[0]
        ai[b, :c] = idx[b, :c]
        ai[b, c:c + len(inblock)] = b * bm + inblock
        am[b, :, :c] = emask[b, :, :c]
        am[b, :, c:c + len(inblock)] = bmask[b][:, inblock]
        assert bmask[b].diagonal().all()
        leaf = np.ones(bm, bool)
        leaf[inblock] = False
        li[b, leaf] = b * bm + np.nonzero(leaf)[0]
    return count, ai, am, li


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
