"""Partition + all-gather logic on two CPU ranks (gloo).  The attention itself is injected (the
oracle stands in); the product's compute path stays CUDA-only."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fstattention_b200 import configs, sharding


def test_shard_bounds_cover_and_balance():
    for n in (1, 5, 64, 67):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def _oracle_attention(q, k, v, meta, sm_scale):
    from oracle import tree_oracle as orc
    out = torch.empty_like(q)
    for z in range(q.shape[0]):
        par = meta[z] if len(meta) > 1 else meta[0]
        lin, _ = orc.lineage_from_parent(par)
        mask = orc.full_attention_mask(lin, pad_rows=0)
        out[z:z + 1] = orc.dense_tree_attention(q[z:z + 1], k[z:z + 1], v[z:z + 1], mask, sm_scale)
    return out


def _worker(rank, world, port, axis, n_trees, heads, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        trees = configs.jittered_forest(1, n_trees, 48)
        g = torch.Generator().manual_seed(0)
        q, k, v = (torch.randn((n_trees, heads, 48, 16), generator=g) for _ in range(3))
        full = _oracle_attention(q, k, v, trees, 0.25)
        ql, kl, vl = (sharding.local_slice(t, axis, world, rank) for t in (q, k, v))
        if axis == "tree":
            lo, hi = sharding.shard_bounds(n_trees, world, rank)
            meta, total = trees[lo:hi], n_trees
        else:
            meta, total = trees, heads
        got = sharding.sharded_fst_attention(ql, kl, vl, meta, 0.25, axis, total,
                                             attention=lambda a, b, c, m, sm_scale: _oracle_attention(a, b, c, m, sm_scale))
        assert got.shape == full.shape
        assert torch.equal(got, full), (axis, rank)
        local_only = sharding.sharded_fst_attention(ql, kl, vl, meta, 0.25, axis, total, gather=False,
                                                    attention=lambda a, b, c, m, sm_scale: _oracle_attention(a, b, c, m, sm_scale))
        assert torch.equal(local_only, sharding.local_slice(full, axis, world, rank))
        # into a caller's buffer; and, where the shards are equal and contiguous in the full
        # tensor, with the collective returned still under way
        buf = torch.empty_like(full)
        inject = lambda a, b, c, m, sm_scale: _oracle_attention(a, b, c, m, sm_scale)
        if total % world == 0 and (axis == "tree" or n_trees == 1):
            got2, work = sharding.sharded_fst_attention(ql, kl, vl, meta, 0.25, axis, total, gathered=buf,
                                                        async_gather=True, attention=inject)
            work.wait()
        else:
            got2 = sharding.sharded_fst_attention(ql, kl, vl, meta, 0.25, axis, total, gathered=buf, attention=inject)
            with pytest.raises(ValueError):
                sharding.all_gather_outputs(local_only, axis, total, async_op=True)
        assert got2 is buf and torch.equal(buf, full)
        open(os.path.join(result_dir, f"ok_{axis}_{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("axis,n_trees,heads", [("tree", 4, 2), ("tree", 5, 2), ("head", 1, 4), ("head", 2, 3)])
def test_two_rank_gather_matches_single_process(tmp_path, axis, n_trees, heads):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), axis, n_trees, heads, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok_{axis}_{r}").exists() for r in range(world))
