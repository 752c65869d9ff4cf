"""The sharded path on real GPUs (needs two): CUDA kernels on every rank's shard, NCCL all-gather
of the outputs, compared with the same problem computed on one GPU and with the CPU oracle."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist
    import fstattention_b200 as fst
    from fstattention_b200 import configs, sharding
    from oracle import tree_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        dev = torch.device("cuda", rank)
        for axis, trees, H in (("tree", configs.jittered_forest(3, 6, 256), 4), ("head", [configs.deep_chain_tree(0, 1024)], 8),
                               ("tree", configs.jittered_forest(4, 5, 256), 2)):      # five trees: shards of three and two
            T, N, D = len(trees), len(trees[0]), 128
            g = torch.Generator().manual_seed(5)
            q, k, v = (torch.randn((T, H, N, D), generator=g).half() for _ in range(3))
            total = T if axis == "tree" else H
            ql, kl, vl = (sharding.local_slice(t, axis, world, rank).contiguous().to(dev) for t in (q, k, v))
            lo, hi = sharding.shard_bounds(total, world, rank)
            mine = trees[lo:hi] if axis == "tree" else trees
            meta = fst.build_tree_metadata(mine if len(mine) > 1 else mine[0], 64, 128)
            full = torch.empty((T, H, N, D), dtype=torch.float16, device=dev)
            if total % world == 0:
                got, work = sharding.sharded_fst_attention(ql, kl, vl, meta, D ** -0.5, axis, total, gathered=full,
                                                           async_gather=True)
                work.wait()
            else:                                        # unequal shards: NCCL gathers padded shards and trims
                got = sharding.sharded_fst_attention(ql, kl, vl, meta, D ** -0.5, axis, total, gathered=full)
            torch.cuda.synchronize()
            # one GPU, whole problem
            meta_all = fst.build_tree_metadata(trees if T > 1 else trees[0], 64, 128)
            single = fst.fst_attention(q.to(dev), k.to(dev), v.to(dev), meta_all, sm_scale=D ** -0.5)
            assert torch.equal(got, single), (axis, rank)
            # the same with the gather done by the attention kernel: every CTA stores its tile
            # into both ranks' copies of the full tensor, then the ranks meet on the stream
            shared = sharding.GatheredOutput((T, H, N, D), torch.float16, dev)
            shared.local.fill_(float("nan"))
            shared.meet()
            fused = sharding.sharded_fst_attention(ql, kl, vl, meta, D ** -0.5, axis, total, scatter_to=shared)
            torch.cuda.synchronize()
            assert fused.data_ptr() == shared.local.data_ptr()
            assert torch.equal(fused, single), (axis, rank, "fused")
            shared.meet()
            if rank == 0:
                t = T - 1
                lin, _ = orc.lineage_from_parent(trees[t])
                mask = orc.full_attention_mask(lin, pad_rows=0)
                exact = orc.dense_tree_attention(q[t:t + 1, -2:], k[t:t + 1, -2:], v[t:t + 1, -2:], mask, D ** -0.5,
                                                 torch.float32)
                assert (got[t:t + 1, -2:].cpu().float() - exact).abs().max().item() <= 2e-3
            assert fst.last_status(dev) == 0
        open(os.path.join(result_dir, f"ok_{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_shards_equal_one_gpu(built_lib, tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"ok_{r}").exists() for r in range(2))
