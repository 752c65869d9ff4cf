"""Tree precompute: the reference's ``utils.py`` surface on top of the CUDA precompute kernel.

``create_fst_attention_kernel_inputs`` keeps the reference's name, arguments, return order,
dtypes and shapes (utils.py:104-129 of the reference) and raises ``RuntimeError`` where the
reference does (more unique ancestors in a block than ``max_ancestors``, utils.py:120), but the
work is done by one kernel launch on the GPU and the tensors it returns live there.
``build_tree_metadata`` is the front door for callers that hold a parent array, which is what a
decoder that rebuilds its tree every step has.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import torch

from . import _lib

TreeLike = Union[torch.Tensor, Sequence[int], Sequence[Sequence[int]]]

# Same tables as the reference's utils.py:4-24: tree depth that fills a context of 2^k - 4 nodes,
# and the ancestor bound its benchmark uses for it.
DEPTH_MAPPING = {2 ** (10 + i): 7 + i for i in range(8)}
MAX_ANCESTOR_MAPPING = {2 ** (10 + i): 64 for i in range(8)}


class TreeMetadata:
    """Block metadata of one tree or a batch of trees, resident on one GPU.

    Unpacks like the reference's return value: ``ancestor_idx, ancestor_mask, leaf_idx = meta``
    (int64 / bool / int64; a leading tree dimension is present only for a batch of trees).
    ``packed`` is the bit-packed form the attention kernels read; ``fst_attention`` accepts the
    object itself in place of the three tensors.
    """

    def __init__(self, n_trees, n_nodes, block_m, max_ancestors, packed, tree_stride, status,
                 ancestor_idx=None, ancestor_mask=None, leaf_idx=None, batched=False):
        self.n_trees, self.n_nodes = n_trees, n_nodes
        self.block_m, self.max_ancestors = block_m, max_ancestors
        self.n_blocks = math.ceil(n_nodes / block_m)
        self.packed, self.tree_stride, self.status = packed, tree_stride, status
        self.ancestor_idx, self.ancestor_mask, self.leaf_idx = ancestor_idx, ancestor_mask, leaf_idx
        self.batched = batched
        self._versions = self._current_versions()
        # attention launches that have read the packed form since it was last written: from the
        # second one on, the launch ahead of the call in the stream cannot be the writer
        self.reads_since_build = 0

    def _current_versions(self):
        return tuple(t._version if t is not None else -1
                     for t in (self.ancestor_idx, self.ancestor_mask, self.leaf_idx))

    def tensors_untouched(self) -> bool:
        """True while nobody has modified the three reference-format tensors in place."""
        return self._versions == self._current_versions()

    def __iter__(self):
        if self.ancestor_idx is None:
            raise RuntimeError("metadata was built with reference_format=False")
        return iter((self.ancestor_idx, self.ancestor_mask, self.leaf_idx))

    def check(self) -> "TreeMetadata":
        """Read the device status record (synchronises) and raise on a recorded problem."""
        code, where, detail, _ = self.status.tolist()
        if code == _lib.DEV_ANCESTOR_OVERFLOW:
            raise RuntimeError(
                f"block {where % 65536} of tree {where // 65536} has {detail} unique ancestors, "
                f"more than max_ancestors={self.max_ancestors}")
        if code == _lib.DEV_MALFORMED_TREE:
            raise ValueError(f"malformed tree: parent[{where}]={detail} must be -1 or an earlier node")
        if code != 0:
            raise RuntimeError(_lib.status_string(code))
        return self

    @property
    def device(self):
        return self.packed.device


# The three tensors handed out by the precompute remember the metadata they came from, so that
# fst_attention(q, k, v, ancestor_idx, ancestor_mask, leaf_idx, ...) can skip re-packing them.
_ORIGIN_ATTR = "_fst_tree_metadata"


def metadata_of(ancestor_idx, ancestor_mask, leaf_idx) -> Optional[TreeMetadata]:
    meta = getattr(ancestor_idx, _ORIGIN_ATTR, None)
    if (meta is not None and meta.ancestor_idx is ancestor_idx and meta.ancestor_mask is ancestor_mask
            and meta.leaf_idx is leaf_idx and meta.tensors_untouched()):
        return meta
    return None


def _as_parent_tensor(parent: TreeLike, device) -> torch.Tensor:
    if not torch.is_tensor(parent):
        parent = torch.tensor(parent, dtype=torch.int32)
    if parent.dim() not in (1, 2) or parent.numel() == 0:
        raise ValueError("parent must be a non-empty [N] or [T, N] array")
    return parent.to(device=device, dtype=torch.int32, non_blocking=True).contiguous()


def packed_meta_bytes(n_blocks: int, block_m: int, max_ancestors: int) -> int:
    return int(_lib.lib().fst_packed_meta_bytes(n_blocks, block_m, max_ancestors))


def build_tree_metadata(parent: TreeLike, block_m: int = 64, max_ancestors: int = 32, *,
                        reference_format: bool = True, check: bool = True,
                        device: Union[str, torch.device, None] = None,
                        out: Optional[TreeMetadata] = None) -> TreeMetadata:
    """Parent array(s) -> block metadata, with one kernel launch on the current stream.

    ``parent`` is ``[N]`` (one tree) or ``[T, N]`` (T independent trees of N nodes); entries are
    -1 for roots and otherwise the index of an earlier node.  ``reference_format=False`` skips
    the int64/bool tensors and writes only the packed form.  ``check=False`` skips reading the
    status record, which avoids a device synchronisation; call ``.check()`` later.  ``out``
    reuses the buffers of an earlier result of the same shape (nothing is allocated then).
    """
    if device is None:
        device = parent.device if torch.is_tensor(parent) and parent.is_cuda else "cuda"
    par = _as_parent_tensor(parent, device)
    batched = par.dim() == 2
    n_trees, n_nodes = (par.shape if batched else (1, par.shape[0]))
    nb = math.ceil(n_nodes / block_m)
    lib = _lib.lib()
    dev = par.device
    if out is not None:
        if (out.n_trees, out.n_nodes, out.block_m, out.max_ancestors) != (n_trees, n_nodes, block_m, max_ancestors):
            raise ValueError("out= metadata has a different shape")
        meta = out
        meta.status.zero_()
    else:
        stride = packed_meta_bytes(nb, block_m, max_ancestors)
        if stride == 0:
            raise ValueError("block_m and max_ancestors must be positive")
        packed = torch.empty((n_trees, stride), dtype=torch.uint8, device=dev)
        status = torch.zeros(_lib.STATUS_WORDS, dtype=torch.int32, device=dev)
        ai = am = li = None
        if reference_format:
            lead = (n_trees,) if batched else ()
            ai = torch.empty(lead + (nb, max_ancestors), dtype=torch.long, device=dev)
            am = torch.empty(lead + (nb, block_m, max_ancestors), dtype=torch.bool, device=dev)
            li = torch.empty(lead + (nb, block_m), dtype=torch.long, device=dev)
        meta = TreeMetadata(n_trees, n_nodes, block_m, max_ancestors, packed, stride, status,
                            ai, am, li, batched)
        if reference_format:
            setattr(ai, _ORIGIN_ATTR, meta)
    with torch.cuda.device(dev):
        rc = lib.fst_precompute(
            par.data_ptr(), n_trees, n_nodes, block_m, max_ancestors,
            meta.ancestor_idx.data_ptr() if meta.ancestor_idx is not None else None,
            meta.ancestor_mask.data_ptr() if meta.ancestor_mask is not None else None,
            meta.leaf_idx.data_ptr() if meta.leaf_idx is not None else None,
            meta.packed.data_ptr(), meta.tree_stride, meta.status.data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "fst_precompute")
    meta._versions = meta._current_versions()
    meta.reads_since_build = 0
    if check:
        meta.check()
    return meta


def tree_topk_nodes(depth: int = 7, topk: int = 4, left_weight_factor: float = 0.5) -> int:
    """Node count of the forest ``build_tree_topk`` / the reference's ``create_tree`` makes."""
    n = int(_lib.lib().fst_tree_topk_nodes(depth, topk, float(left_weight_factor)))
    if n < 0:
        raise ValueError("forest shape beyond the kernel's limits (a level above 4096 nodes, or more than 32 levels)")
    return n


def build_tree_topk(scores: torch.Tensor, depth: Optional[int] = None, topk: Optional[int] = None,
                    left_weight_factor: float = 0.5, max_nodes: Optional[int] = None, *,
                    return_choice: bool = False, return_scores: bool = False):
    """Grow the speculation tree on the GPU from the heads' top-k candidate scores.

    ``scores`` is a CUDA float32 tensor ``[depth + 1, topk]`` (one tree) or ``[T, depth + 1, topk]``:
    row ``l`` holds the scores (log-probabilities) of head ``l``'s ``topk`` candidates.  The
    forest has the shape of the reference's ``create_tree(depth, topk, left_weight_factor)``
    (utils.py:27-77) - ``topk`` roots, of every level the ``int(size * left_weight_factor)``
    best-scoring nodes (score = sum along the path) expanded into the next head's candidates -
    and with equal scores is exactly that forest.  Returns the parent array, int32 ``[N]`` /
    ``[T, N]`` on the GPU (``N = max_nodes`` or the forest's node count), ready for
    ``dfs_order_device`` / ``build_tree_metadata(parent, check=False)``; with ``return_choice``
    also ``choice`` (``l * topk + k``: which candidate each node stands for) and with
    ``return_scores`` the nodes' path scores.  One launch on the current stream, no host
    synchronisation.
    """
    if not scores.is_cuda or scores.dtype != torch.float32 or scores.dim() not in (2, 3):
        raise TypeError("scores must be a CUDA float32 tensor [depth + 1, topk] or [T, depth + 1, topk]")
    batched = scores.dim() == 3
    levels, k = scores.shape[-2:]
    depth = levels - 1 if depth is None else depth
    topk = k if topk is None else topk
    if (depth + 1, topk) != (levels, k):
        raise ValueError("scores must have depth + 1 rows of topk entries")
    n_trees = scores.shape[0] if batched else 1
    total = tree_topk_nodes(depth, topk, left_weight_factor)
    n = total if max_nodes is None else int(max_nodes)
    if n <= 0:
        raise ValueError("max_nodes must be positive")
    sc = scores.contiguous()
    dev = sc.device
    lead = (n_trees,) if batched else ()
    parent = torch.empty(lead + (n,), dtype=torch.int32, device=dev)
    choice = torch.empty(lead + (n,), dtype=torch.int32, device=dev) if return_choice else None
    nscore = torch.empty(lead + (n,), dtype=torch.float32, device=dev) if return_scores else None
    with torch.cuda.device(dev):
        rc = _lib.lib().fst_build_tree_topk(
            sc.data_ptr(), n_trees, depth, topk, float(left_weight_factor), n, parent.data_ptr(),
            choice.data_ptr() if choice is not None else None,
            nscore.data_ptr() if nscore is not None else None,
            torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "fst_build_tree_topk")
    extra = tuple(t for t in (choice, nscore) if t is not None)
    return (parent,) + extra if extra else parent


def parent_from_lineage(lineage: torch.Tensor, level_lookup: torch.Tensor) -> torch.Tensor:
    """parent[k] = lineage[k, level_lookup[k] - 1], -1 for level-0 nodes (utils.py:42-44)."""
    lvl = level_lookup.to(lineage.device).long()
    col = (lvl - 1).clamp_min(0).unsqueeze(1)
    par = lineage.gather(1, col).squeeze(1)
    return torch.where(lvl > 0, par, torch.full_like(par, -1))


def create_fst_attention_kernel_inputs(lineage: torch.Tensor, level_lookup: torch.Tensor,
                                       block_m: int = 64, max_ancestors: int = 32,
                                       mutate_lineage: bool = True):
    """Drop-in for the reference function of the same name (utils.py:104-129).

    Returns ``ancestor_idx [nb, max_ancestors]`` (int64), ``ancestor_mask [nb, block_m,
    max_ancestors]`` (bool) and ``leaf_idx [nb, block_m]`` (int64) with the reference's values,
    as CUDA tensors.  Raises RuntimeError when a block has more than ``max_ancestors`` unique
    ancestors.  Like the reference (utils.py:124-125) it writes every node into its own lineage
    row as a side effect; pass ``mutate_lineage=False`` to leave ``lineage`` alone.
    """
    parent = parent_from_lineage(lineage, level_lookup)
    meta = build_tree_metadata(parent, block_m, max_ancestors, reference_format=True, check=True)
    if mutate_lineage:
        n = lineage.shape[0]
        rows = torch.arange(n, device=lineage.device)
        lineage[rows, level_lookup.to(lineage.device).long()] = rows
    return meta.ancestor_idx, meta.ancestor_mask, meta.leaf_idx


def lineage_from_parent(parent: Sequence[int]):
    """Parent array -> (lineage, level_lookup) as the reference describes trees (utils.py:42-44).

    Host-side adapter for callers that still want the reference's inputs; CPU tensors.
    """
    n = len(parent)
    level = [0] * n
    for i, p in enumerate(parent):
        if p >= i or p < -1:
            raise ValueError(f"parent[{i}]={p} must be -1 or an earlier node")
        level[i] = 0 if p < 0 else level[p] + 1
    width = max(level) + 1
    lin = torch.full((n, width), -1, dtype=torch.long)
    for i, p in enumerate(parent):
        if p >= 0:
            lin[i, : level[p]] = lin[p, : level[p]]
            lin[i, level[p]] = p
    return lin, torch.tensor(level, dtype=torch.long)


def create_tree(depth: int = 7, topk: int = 4, left_weight_factor: float = 0.5):
    """The reference's synthetic left-weighted forest (utils.py:27-77), built without loops over
    nodes.

    ``topk`` roots; level sizes follow ``size[l] = topk * int(size[l-1] * left_weight_factor)``
    and node ``r`` of a level hangs under node ``r // topk`` of the level above.  With the
    defaults the forest has 2^(depth+3) - 4 nodes.  Returns ``lineage [N, depth + 1]`` (ancestor
    of each node per level, -1 padded, the node itself not included) and ``level_lookup [N]``,
    both int64 on the CPU, equal to what the reference returns.
    """
    sizes = [topk]
    for _ in range(depth):
        sizes.append(topk * int(sizes[-1] * left_weight_factor))
    starts = [0]
    for sz in sizes:
        starts.append(starts[-1] + sz)
    n = starts[-1]
    level = torch.repeat_interleave(torch.arange(len(sizes)), torch.tensor(sizes))
    start_of = torch.tensor(starts[:-1])[level]
    rel = torch.arange(n) - start_of
    parent = torch.where(level > 0, torch.tensor([0] + starts[:-2])[level] + rel // topk,
                         torch.full((n,), -1, dtype=torch.long))
    lineage = torch.full((n, depth + 1), -1, dtype=torch.long)
    anc = parent.clone()
    for step in range(1, depth + 1):                     # ancestor `step` levels up, all nodes at once
        has = anc >= 0
        rows = torch.nonzero(has).squeeze(1)
        lineage[rows, level[rows] - step] = anc[rows]
        anc = torch.where(has, parent[anc.clamp_min(0)], anc)
    return lineage, level.long()


def create_full_attention_mask(lineage: torch.Tensor) -> torch.Tensor:
    """Dense mask "node attends to itself and its ancestors", as the reference builds it
    (utils.py:79-102), on the device ``lineage`` lives on.

    float32 ``[N + 4, N + 4]``: the reference always appends four zero rows and columns (its
    trees have 2^k - 4 nodes), clears the last column while removing the -1 pads and restores
    only the last node's self entry.  For other sizes pad ``mask[:N, :N]`` yourself.
    """
    n = lineage.shape[0]
    dev = lineage.device
    mask = torch.zeros((n, n), dtype=torch.bool, device=dev)
    rows = torch.arange(n, device=dev).unsqueeze(1).expand_as(lineage)
    mask[rows.reshape(-1), lineage.reshape(-1)] = True    # -1 lands in the last column
    mask[torch.arange(n, device=dev), torch.arange(n, device=dev)] = True
    mask[:, -1] = False
    mask[-1, -1] = True
    out = torch.zeros((n + 4, n + 4), dtype=torch.float32, device=dev)
    out[:n, :n] = mask
    return out


def dfs_order(parent: Sequence[int]):
    """Depth-first renumbering of a tree, so that a query block's ancestors are few and local.

    The reference leaves this as a TODO (README.md:19-20): with nodes numbered breadth first a
    block of 64 rows of a deep tree has ancestors all over the tree (a 2579-node chain tree needs
    up to 1613 per block and gathers 8x the bytes); numbered depth first, a block is a few
    root-to-leaf paths.  Returns ``(order, new_parent)``: ``order[i]`` is the old index of the
    node that becomes node ``i`` (pre-order, children in their old relative order) and
    ``new_parent`` is the parent array in the new numbering, still with ``new_parent[i] < i``.
    Permute the tree rows of q/k/v with ``order`` (``x[..., order, :]``) before attention and
    scatter the output back (``out[..., order, :] = o``).  Host code (numpy); trees are small.
    """
    import numpy as np
    par = np.asarray(parent, dtype=np.int64)
    n = par.shape[0]
    if n == 0:
        return [], []
    if np.any(par >= np.arange(n)) or np.any(par < -1):
        raise ValueError("parent[i] must be -1 or an earlier node")
    size = np.ones(n, dtype=np.int64)
    for i in range(n - 1, -1, -1):                       # children come after parents
        if par[i] >= 0:
            size[par[i]] += size[i]
    # position = position of parent + 1 + sizes of earlier siblings; roots are siblings of each other
    pos = np.empty(n, dtype=np.int64)
    next_free = {}                                       # parent (or -1) -> next free position
    for i in range(n):
        p = int(par[i])
        start = next_free.get(p, 0 if p < 0 else pos[p] + 1)
        pos[i] = start
        next_free[p] = start + size[i]
    order = np.empty(n, dtype=np.int64)
    order[pos] = np.arange(n)
    new_parent = np.where(par[order] >= 0, pos[np.clip(par[order], 0, None)], -1)
    return order.tolist(), new_parent.tolist()


def dfs_order_device(parent: TreeLike, *, check: bool = True,
                     device: Union[str, torch.device, None] = None):
    """``dfs_order`` computed on the GPU with one kernel launch on the current stream, for parent
    arrays that already live there (a decoder that builds its tree on the device).

    ``parent`` is ``[N]`` or ``[T, N]`` as for ``build_tree_metadata`` (N <= 8192).  Returns
    ``(order, new_parent)`` as int32 CUDA tensors of the same shape, with the meaning
    ``dfs_order`` gives them; ``new_parent`` goes straight into ``build_tree_metadata``.
    ``check=False`` skips reading the status record (no device synchronisation); a malformed
    tree then leaves both outputs uninitialised."""
    if device is None:
        device = parent.device if torch.is_tensor(parent) and parent.is_cuda else "cuda"
    par = _as_parent_tensor(parent, device)
    n_trees, n_nodes = (par.shape if par.dim() == 2 else (1, par.shape[0]))
    order = torch.empty_like(par)
    new_parent = torch.empty_like(par)
    status = torch.zeros(_lib.STATUS_WORDS, dtype=torch.int32, device=par.device)
    with torch.cuda.device(par.device):
        rc = _lib.lib().fst_dfs_order(par.data_ptr(), n_trees, n_nodes, order.data_ptr(), new_parent.data_ptr(),
                                      status.data_ptr(), torch.cuda.current_stream(par.device).cuda_stream)
    _lib.check(rc, "fst_dfs_order")
    if check:
        code, where, detail, _ = status.tolist()
        if code == _lib.DEV_MALFORMED_TREE:
            raise ValueError(f"parent[{where}] = {detail} is neither -1 nor an earlier node")
        if code != 0:
            raise RuntimeError(f"fst_dfs_order: device status {code}")
    return order, new_parent

