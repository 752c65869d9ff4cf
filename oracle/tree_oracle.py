"""CPU oracle for the tree-attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU with torch/numpy, what the reference computes for the path
"block-metadata precompute + tree-masked attention".  It exists so that the CUDA kernels can be
checked against it; the product never imports it (only the tests, the smoke check and the CPU
baseline leg of the benchmark do).

Parity status: PINNED.  ``tests/golden/`` holds metadata produced by the reference's own
``utils.create_fst_attention_kernel_inputs`` / ``create_full_attention_mask`` and attention
outputs produced by the reference's own Triton kernel (run under the Triton CPU interpreter) and
by its dense formula; ``tests/test_oracle_golden.py`` checks every function below against them.

Reference locations restated here (paths inside the reference project):
  * lineage / level_lookup contract ........ utils.py:42-44, 66-77
  * dense full mask ......................... utils.py:79-102
  * block metadata .......................... utils.py:104-129
  * dense tree-masked attention ............. fstattention.py:214-219 (prefix: 207-212)
"""
from __future__ import annotations

import math
from typing import Sequence, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------------------------
# parent array  <->  lineage / level_lookup            (input contract, utils.py:42-44, 66-77)
# --------------------------------------------------------------------------------------------
def lineage_from_parent(parent: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Build the reference's tree description from a parent array.

    ``lineage[k, l]`` is the ancestor of node ``k`` at level ``l`` (roots are level 0) and -1
    elsewhere; the node itself is not included.  ``level_lookup[k]`` is the level of ``k``.
    The width is ``max_level + 1`` so every row keeps at least one -1, which the reference's
    ``unique(...)[1:]`` relies on (utils.py:119).
    """
    par = np.asarray(parent, dtype=np.int64)
    n = par.shape[0]
    level = np.zeros(n, dtype=np.int64)
    for i in range(n):
        p = par[i]
        if p >= i or p < -1:
            raise ValueError(f"parent[{i}]={p} must be -1 or an earlier node")
        level[i] = 0 if p < 0 else level[p] + 1
    width = int(level.max()) + 1 if n else 1
    lin = np.full((n, width), -1, dtype=np.int64)
    for i in range(n):
        p = par[i]
        if p >= 0:
            lin[i, : level[p]] = lin[p, : level[p]]
            lin[i, level[p]] = p
    return torch.from_numpy(lin), torch.from_numpy(level)


def parent_from_lineage(lineage: torch.Tensor, level_lookup: torch.Tensor) -> torch.Tensor:
    """Inverse adapter: parent[k] = lineage[k, level[k]-1], -1 for level-0 nodes."""
    lin = lineage.cpu().numpy()
    lvl = level_lookup.cpu().numpy()
    n = lin.shape[0]
    par = np.full(n, -1, dtype=np.int64)
    nz = lvl > 0
    par[nz] = lin[np.arange(n)[nz], lvl[nz] - 1]
    return torch.from_numpy(par)


# --------------------------------------------------------------------------------------------
# dense full mask                                                          (utils.py:79-102)
# --------------------------------------------------------------------------------------------
def full_attention_mask(lineage: torch.Tensor, pad_rows: int | None = 4) -> torch.Tensor:
    """Dense 0/1 mask "node attends to itself and to its ancestors", float32.

    Follows utils.py:87-100: scatter each lineage row (its -1 pads land in the last column),
    set the diagonal, clear the last column, restore the last node's self entry, then append
    ``pad_rows`` zero rows and columns.  The reference hard-codes ``pad_rows=4`` (its trees have
    2^k-4 nodes); pass the amount that rounds N up to a multiple of the query block otherwise,
    or ``None``/0 for no padding.
    """
    lin = lineage.cpu().numpy()
    n = lin.shape[0]
    m = np.zeros((n, n), dtype=bool)
    rows = np.repeat(np.arange(n), lin.shape[1])
    m[rows, lin.reshape(-1)] = True            # -1 indexes the last column, as in the reference
    m[np.arange(n), np.arange(n)] = True
    m[:, -1] = False
    m[-1, -1] = True
    pad = int(pad_rows or 0)
    out = np.zeros((n + pad, n + pad), dtype=np.float32)
    out[:n, :n] = m
    return torch.from_numpy(out)


def block_padded_mask(lineage: torch.Tensor, block_m: int) -> torch.Tensor:
    """Full mask padded to ceil(N/block_m)*block_m rows and columns (pad rows are all zero)."""
    n = lineage.shape[0]
    return full_attention_mask(lineage, pad_rows=(-n) % block_m)


# --------------------------------------------------------------------------------------------
# block metadata                                                          (utils.py:104-129)
# --------------------------------------------------------------------------------------------
def block_metadata(lineage: torch.Tensor, level_lookup: torch.Tensor, block_m: int = 64,
                   max_ancestors: int = 32, blocks: Sequence[int] | None = None):
    """Per query block: sorted unique ancestors, row-by-ancestor mask, leaf list.

    Returns ``(ancestor_idx [nb, MA] int64, ancestor_mask [nb, bm, MA] bool,
    leaf_idx [nb, bm] int64)`` with -1 / False padding, exactly as utils.py:112-129:

      * ancestors of a block = sorted unique non-negative entries of its lineage rows
        (utils.py:119: ``unique`` then drop the leading -1);
      * more than ``max_ancestors`` of them raises RuntimeError (the slice assignment at
        utils.py:120 fails);
      * leaves = {i .. i+block_m-1} minus the block's ancestors, *including* indices past the
        last node in a partial last block (utils.py:121-122);
      * mask[j, a] = ancestor a is in (lineage row j plus the node j itself) for real rows
        (utils.py:124-127).

    Unlike the reference this does not modify ``lineage`` (the reference writes each node into
    its own lineage row, utils.py:124-125); the caller's tensor is left alone.  ``blocks``
    restricts the loop of utils.py:114 to the listed blocks (spot checks of very large trees);
    the other blocks' entries keep their padding values.
    """
    n = lineage.shape[0]
    nb = math.ceil(n / block_m)
    anc_idx = torch.full((nb, max_ancestors), -1, dtype=torch.long)
    anc_mask = torch.zeros((nb, block_m, max_ancestors), dtype=torch.bool)
    leaf_idx = torch.full((nb, block_m), -1, dtype=torch.long)
    lin = lineage.clone()
    for b in (range(nb) if blocks is None else blocks):
        lo, hi = b * block_m, min((b + 1) * block_m, n)
        rows = lin[lo:hi]
        uniq = torch.unique(rows.reshape(-1))
        uniq = uniq[1:]                                   # drop the -1 pad (smallest value)
        cnt = uniq.shape[0]
        if cnt > max_ancestors:
            raise RuntimeError(
                f"block {b} has {cnt} unique ancestors, more than max_ancestors={max_ancestors}")
        anc_idx[b, :cnt] = uniq
        in_block = set(range(lo, lo + block_m))
        for k in sorted(in_block.difference(uniq.tolist())):
            leaf_idx[b, k - lo] = k
        for k in range(lo, hi):
            with_self = torch.cat((rows[k - lo], torch.tensor([k], dtype=torch.long)))
            anc_mask[b, k - lo, :cnt] = torch.isin(uniq, with_self)
    return anc_idx, anc_mask, leaf_idx


def block_metadata_from_parent(parent: Sequence[int], block_m: int, max_ancestors: int):
    lin, lvl = lineage_from_parent(parent)
    return block_metadata(lin, lvl, block_m, max_ancestors)


def gathered_rows(ancestor_idx: torch.Tensor, leaf_idx: torch.Tensor, n_nodes: int) -> int:
    """Rows of K (and of V) one head gathers: valid ancestors + leaves that are real nodes."""
    a = int((ancestor_idx >= 0).sum())
    l = int(((leaf_idx >= 0) & (leaf_idx < n_nodes)).sum())
    return a + l


# --------------------------------------------------------------------------------------------
# dense tree-masked attention                                       (fstattention.py:214-219)
# --------------------------------------------------------------------------------------------
def dense_tree_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                         sm_scale: float, compute_dtype: torch.dtype | None = None,
                         head_chunk: int | None = None) -> torch.Tensor:
    """softmax(mask(Q K^T * scale)) V as the reference's test writes it.

    Scores are formed in the input dtype, entries with ``mask == 0`` become -inf, the softmax
    runs in float32 and is cast back to the input dtype before the second matmul
    (fstattention.py:216-219).  ``mask`` is ``[Nq, Nkv]`` and shared by every batch element and
    head; with a shared prefix of P rows it is ``[ones(Nq, P) | tree mask]``
    (fstattention.py:209).  Rows whose mask is all zero come out NaN, as in the reference.

    ``compute_dtype`` evaluates the same formula after up-casting the inputs (float32/float64),
    which gives the rounding-free value of the same function.  ``head_chunk`` bounds memory.
    """
    if compute_dtype is not None:
        q, k, v = q.to(compute_dtype), k.to(compute_dtype), v.to(compute_dtype)
    dead = (mask == 0)
    z, h = q.shape[0], q.shape[1]
    out = torch.empty_like(q)
    step = head_chunk or h
    for h0 in range(0, h, step):
        qs, ks, vs = q[:, h0:h0 + step], k[:, h0:h0 + step], v[:, h0:h0 + step]
        p = torch.matmul(qs, ks.transpose(2, 3)) * sm_scale
        p[:, :, dead] = float("-inf")
        soft_dtype = torch.float32 if p.dtype != torch.float64 else torch.float64
        p = torch.softmax(p.to(soft_dtype), dim=-1).to(qs.dtype)
        out[:, h0:h0 + step] = torch.matmul(p, vs)
    return out


def tree_attention_reference(q, k, v, parent: Sequence[int], sm_scale: float, block_m: int,
                             prefix_len: int = 0, compute_dtype=None, head_chunk=None):
    """Dense oracle for one tree given as a parent array; q has nb*block_m (padded) rows."""
    lin, _ = lineage_from_parent(parent)
    mask = block_padded_mask(lin, block_m)
    nq = q.shape[2]
    if mask.shape[0] < nq:                      # caller padded further
        big = torch.zeros((nq, nq))
        big[: mask.shape[0], : mask.shape[1]] = mask
        mask = big
    if prefix_len:
        mask = torch.cat((torch.ones((mask.shape[0], prefix_len)), mask), dim=1)
    return dense_tree_attention(q, k, v, mask, sm_scale, compute_dtype, head_chunk)
