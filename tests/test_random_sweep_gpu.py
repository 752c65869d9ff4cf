"""Seeded random sweeps over shapes the other tests do not name one by one."""
import random

import pytest
import torch

from oracle import tree_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fst(built_lib):
    import fstattention_b200
    return fstattention_b200


def test_random_forests_metadata_order_and_attention(fst):
    """Random forests (windows from chains to wide fans, stray extra roots), every block size: the
    device renumbering equals the host one, the metadata equals the oracle's bit for bit, and the
    tensor-core kernel agrees with the fp32 kernel."""
    rng = random.Random(11)
    for it in range(120):
        n = rng.randint(1, 1500)
        win = rng.choice([1, 3, 16, 64, 400])
        par = [-1] + [rng.randint(-1 if rng.random() < 0.02 else max(0, i - win), i - 1) for i in range(1, n)]
        order, new_parent = fst.dfs_order(par)
        d_order, d_parent = fst.dfs_order_device(par)
        assert d_order.cpu().tolist() == order and d_parent.cpu().tolist() == new_parent, (it, n, win)
        bm = rng.choice([16, 32, 64, 128])
        ai, am, li = orc.block_metadata_from_parent(par, bm, 2048)
        meta = fst.build_tree_metadata(par, bm, 2048)
        assert torch.equal(meta.ancestor_idx.cpu(), ai), (it, n, win, bm)
        assert torch.equal(meta.ancestor_mask.cpu(), am), (it, n, win, bm)
        assert torch.equal(meta.leaf_idx.cpu(), li), (it, n, win, bm)
        if it % 4 == 0 and bm >= 32:
            D, H = rng.choice([64, 128]), rng.randint(1, 4)
            g = torch.Generator(device="cuda").manual_seed(it)
            q, k, v = (torch.randn((1, H, n, D), generator=g, device="cuda").half() for _ in range(3))
            fast = fst.fst_attention(q, k, v, meta, sm_scale=D ** -0.5)
            exact = fst.fst_attention(q.float(), k.float(), v.float(), meta, sm_scale=D ** -0.5, kernel="simt")
            assert (fast.float() - exact).abs().max().item() <= 2e-3, (it, n, win, bm, D)
    assert fst.last_status() == 0


def test_random_prefix_shapes_on_the_tcgen05_path(fst):
    """Random (head_dim, dtype, tree size, prefix length, heads, K/V heads, batch, runs, block size):
    the tcgen05 prefix path agrees with the tree kernel walking the prefix in one piece, and gives
    the same bits when called again (every hand-off in it is a barrier, none a matter of timing)."""
    from fstattention_b200 import configs
    rng = random.Random(7)
    for it in range(150):
        D = rng.choice([64, 128])
        dtype = rng.choice([torch.float16, torch.bfloat16])
        n = rng.choice([64, 100, 256, 300, 512])
        prefix, H, Z = rng.randint(1, 5000), rng.randint(1, 6), rng.randint(1, 3)
        H_kv = rng.choice([h for h in range(1, H + 1) if H % h == 0])
        runs, bm = rng.randint(1, 5), rng.choice([32, 64, 128])
        par = configs.random_window_tree(rng.randint(0, 10 ** 6), n, rng.choice([8, 40]))
        meta = fst.build_tree_metadata(par, bm, 512, reference_format=False)
        g = torch.Generator(device="cuda").manual_seed(it)
        q = torch.randn((Z, H, n, D), generator=g, device="cuda").to(dtype)
        k = torch.randn((Z, H_kv, prefix + n, D), generator=g, device="cuda").to(dtype)
        v = torch.randn((Z, H_kv, prefix + n, D), generator=g, device="cuda").to(dtype)
        scale = D ** -0.5
        a, la = fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_umma", kv_splits=runs, return_lse=True)
        b, lb = fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_t32", kv_splits=1, return_lse=True)
        again = fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_umma", kv_splits=runs)
        what = (it, D, dtype, n, prefix, H, H_kv, Z, runs, bm)
        assert torch.equal(a, again), what
        assert torch.isfinite(a).all(), what
        assert (a.float() - b.float()).abs().max().item() <= (2e-3 if dtype == torch.float16 else 1.6e-2), what
        assert (la - lb).abs().max().item() <= 2e-2, what
    assert fst.last_status() == 0
