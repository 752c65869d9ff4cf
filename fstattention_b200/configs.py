"""Workload definitions: the token trees and tensor shapes the kernels are measured on.

Every tree is a *parent array*: ``parent[i]`` is the index of node ``i``'s parent, ``-1`` for a
root, and parents always precede their children (``parent[i] < i``).  The reference describes
trees by a ``lineage`` matrix and a ``level_lookup`` vector (utils.py:42-44 of the reference);
``lineage_from_parent`` in this package converts between the two.

All inputs are synthetic and seeded; nothing here reads a dataset.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import List, Sequence

MEDUSA_FANOUT = (10, 8, 6, 4, 3, 2)


def binary_tree(n: int = 31) -> List[int]:
    """Complete binary tree in BFS order: parent[i] = (i-1)//2."""
    return [-1] + [(i - 1) // 2 for i in range(1, n)]


def left_weighted_tree(fanout: Sequence[int] = MEDUSA_FANOUT, n: int = 256) -> List[int]:
    """Medusa-style static tree, expanded breadth first.

    A node at depth ``d`` whose rank among its siblings is ``r`` (0-based) gets
    ``max(0, fanout[d] - r)`` children (none below ``len(fanout)``); expansion stops once ``n``
    nodes exist.
    """
    parent, depth, rank = [-1], [0], [0]
    head = 0
    while len(parent) < n and head < len(parent):
        d, r = depth[head], rank[head]
        n_child = max(0, fanout[d] - r) if d < len(fanout) else 0
        for j in range(n_child):
            if len(parent) >= n:
                break
            parent.append(head)
            depth.append(d + 1)
            rank.append(j)
        head += 1
    return parent


def random_window_tree(seed: int, n: int = 1024, window: int = 64) -> List[int]:
    """Dynamic tree: parent[i] uniform in [max(0, i-window), i-1]."""
    rng = random.Random(seed)
    return [-1] + [rng.randint(max(0, i - window), i - 1) for i in range(1, n)]


def jittered_forest(seed: int = 0, trees: int = 64, n: int = 256) -> List[List[int]]:
    """Independent left-weighted trees whose per-depth fan-out is jittered by -1/0/+1."""
    rng = random.Random(seed)
    out = []
    for _ in range(trees):
        fan = tuple(max(0, c + rng.choice((-1, 0, 1))) for c in MEDUSA_FANOUT)
        out.append(left_weighted_tree(fan, n))
    return out


def deep_chain_tree(seed: int = 0, n: int = 4096, trunk: int = 32, chain_len: int = 32,
                    chains: int | None = None, sibling_p: float = 0.25) -> List[int]:
    """Deep tree: chains of ``chain_len`` nodes hanging off the last node of a ``trunk`` chain.

    After each chain node a single-leaf sibling (same parent) is added with probability
    ``sibling_p``.  Nodes are numbered in construction order (trunk, then chain by chain, each
    sibling right after its chain node), which keeps a query block's ancestors local.

    With ``chains=None`` chains are added until ``n`` nodes exist and the list is cut at ``n``
    (64 chains alone give only about 2.6k nodes); with ``chains=64`` the tree is the literal
    64-chain one, cut at ``n`` if it is longer.
    """
    rng = random.Random(seed)
    parent = [-1] + list(range(trunk - 1))
    done = 0
    while (chains is None and len(parent) < n) or (chains is not None and done < chains):
        prev = trunk - 1
        for _ in range(chain_len):
            parent.append(prev)
            me = len(parent) - 1
            if rng.random() < sibling_p:
                parent.append(prev)
            prev = me
        done += 1
    return parent[:n]


@dataclass
class Workload:
    """One measurement configuration: trees plus tensor shapes."""
    name: str
    trees: List[List[int]]          # one parent array per independent tree (batch element)
    heads: int
    head_dim: int
    dtype: str                      # "fp16" | "bf16" | "fp32"
    block_m: int
    max_ancestors: int
    shard: str = "none"             # "none" | "tree" | "head"
    prefix: int = 0                 # shared K/V rows every query attends to (the prompt)
    notes: str = ""
    extras: dict = field(default_factory=dict)

    @property
    def n_nodes(self) -> int:
        return len(self.trees[0])

    @property
    def sm_scale(self) -> float:
        return self.head_dim ** -0.5


def workload(name: str, step: int = 0) -> Workload:
    """The five configurations, by name: binary31, medusa256, random1024, forest64, deep4096."""
    if name == "binary31":
        return Workload(name, [binary_tree(31)], heads=4, head_dim=64, dtype="fp32",
                        block_m=16, max_ancestors=16)
    if name == "medusa256":
        return Workload(name, [left_weighted_tree()], heads=32, head_dim=128, dtype="fp16",
                        block_m=64, max_ancestors=64)
    if name == "random1024":
        return Workload(name, [random_window_tree(step)], heads=32, head_dim=128, dtype="fp16",
                        block_m=64, max_ancestors=320,      # seeds 0..99 need up to 257 per block
                        notes="tree regenerated every step; step index is the seed")
    if name == "forest64":
        return Workload(name, jittered_forest(0, 64, 256), heads=32, head_dim=128, dtype="fp16",
                        block_m=64, max_ancestors=64, shard="tree")
    if name == "deep4096":
        return Workload(name, [deep_chain_tree(0, 4096)], heads=64, head_dim=128, dtype="fp16",
                        block_m=64, max_ancestors=128, shard="head")
    if name == "medusa256_prefix4096":
        return Workload(name, [left_weighted_tree()], heads=32, head_dim=128, dtype="fp16",
                        block_m=64, max_ancestors=64, prefix=4096,
                        notes="decode step: 4096-token prompt shared by the 256-node tree")
    raise KeyError(name)


WORKLOADS = ("binary31", "medusa256", "random1024", "forest64", "deep4096")
