"""GPU precompute kernel against the reference's own outputs (golden) and the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import unpack_golden_metadata
from helpers import decode_packed
from oracle import tree_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fst(built_lib):
    import fstattention_b200
    return fstattention_b200


def test_metadata_bit_exact_vs_reference_golden(fst, metadata_golden):
    for name, case in metadata_golden.items():
        ai, am, li, bm, ma = unpack_golden_metadata(case)
        meta = fst.build_tree_metadata(case["parent"].tolist(), bm, ma)
        g_ai, g_am, g_li = meta
        assert g_ai.dtype == torch.long and g_am.dtype == torch.bool and g_li.dtype == torch.long
        assert torch.equal(g_ai.cpu(), ai), name
        assert torch.equal(g_am.cpu(), am), name
        assert torch.equal(g_li.cpu(), li), name
        # the packed form says the same thing
        nb = ai.shape[0]
        cnt, p_idx, p_mask, p_leaf = decode_packed(meta.packed[0].cpu().numpy(), nb, bm, ma)
        lo = torch.arange(nb)[:, None] * bm
        external = (ai >= 0) & ((ai < lo) | (ai >= lo + bm))
        assert np.array_equal(cnt, external.sum(1).numpy()), name
        assert np.array_equal(p_idx, ai.numpy()), name
        assert np.array_equal(p_mask, am.numpy()), name
        assert np.array_equal(p_leaf, li.numpy()), name


def test_packed_only_matches(fst, metadata_golden):
    case = metadata_golden["random1024_s1_bm64"]
    ai, am, li, bm, ma = unpack_golden_metadata(case)
    meta = fst.build_tree_metadata(case["parent"].tolist(), bm, ma, reference_format=False)
    assert meta.ancestor_idx is None
    cnt, p_idx, p_mask, p_leaf = decode_packed(meta.packed[0].cpu().numpy(), ai.shape[0], bm, ma)
    assert np.array_equal(p_idx, ai.numpy()) and np.array_equal(p_mask, am.numpy())
    assert np.array_equal(p_leaf, li.numpy())


def test_batched_forest_vs_oracle(fst):
    from fstattention_b200 import configs
    forest = configs.jittered_forest(0, 64, 256)
    meta = fst.build_tree_metadata(forest, 64, 64)
    g_ai, g_am, g_li = (t.cpu() for t in meta)
    assert g_ai.shape == (64, 4, 64) and g_am.shape == (64, 4, 64, 64) and g_li.shape == (64, 4, 64)
    for t in range(0, 64, 7):
        ai, am, li = orc.block_metadata_from_parent(forest[t], 64, 64)
        assert torch.equal(g_ai[t], ai) and torch.equal(g_am[t], am) and torch.equal(g_li[t], li), t


@pytest.mark.parametrize("seed", range(6))
def test_random_trees_vs_oracle(fst, seed):
    rng = np.random.RandomState(seed)
    n = int(rng.randint(1, 700))
    roots = int(rng.randint(1, 4))
    window = int(rng.choice([2, 8, 64, 10_000]))
    par = [-1] * min(roots, n) + [int(rng.randint(max(0, i - window), i)) for i in range(min(roots, n), n)]
    bm = int(rng.choice([8, 16, 24, 64, 128]))
    ai, am, li = orc.block_metadata_from_parent(par, bm, 4096)
    ma = max(4, int((ai >= 0).sum(1).max()) + int(rng.randint(0, 9)))
    ai, am, li = orc.block_metadata_from_parent(par, bm, ma)
    g_ai, g_am, g_li = (t.cpu() for t in fst.build_tree_metadata(par, bm, ma))
    assert torch.equal(g_ai, ai) and torch.equal(g_am, am) and torch.equal(g_li, li)


def test_large_tree_attention_sets(fst):
    """8192 nodes: every row's metadata set equals {itself} + its parent chain."""
    from fstattention_b200 import configs
    par = configs.random_window_tree(3, 8192, 64)
    bm, ma = 64, 512
    ai, am, li = (t.cpu().numpy() for t in fst.build_tree_metadata(par, bm, ma))
    for b in range(ai.shape[0]):
        row = ai[b][ai[b] >= 0]
        assert np.all(np.diff(row) > 0)                      # ascending, unique
    for k in range(0, 8192, 13):
        b, j = divmod(k, bm)
        got = set(ai[b][am[b, j]].tolist())
        if li[b, j] >= 0:
            assert li[b, j] == k
            got.add(k)
        want, x = {k}, par[k]
        while x >= 0:
            want.add(x)
            x = par[x]
        assert got == want, k


def test_overflow_raises_and_gpu_stays_usable(fst, metadata_golden):
    par = metadata_golden["medusa256_bm64"]["parent"].tolist()
    with pytest.raises(RuntimeError, match="max_ancestors"):
        fst.build_tree_metadata(par, 64, 16)
    meta = fst.build_tree_metadata(par, 64, 16, check=False)     # no sync, no raise
    assert int(meta.status[0].item()) == 17
    # the first 16 ancestors of every block were kept
    ai = orc.block_metadata_from_parent(par, 64, 64)[0]
    assert torch.equal(meta.ancestor_idx.cpu(), ai[:, :16])
    fst.build_tree_metadata(par, 64, 64)                         # still fine afterwards


def test_malformed_parent_is_reported_not_faulted(fst):
    par = [-1, 0, 1, 5, 2, 3]                                    # parent[3] = 5 points forward
    with pytest.raises(ValueError, match="malformed"):
        fst.build_tree_metadata(par, 16, 16)
    with pytest.raises(ValueError, match="malformed"):
        fst.build_tree_metadata([-1, 0, -7, 1], 16, 16)
    fst.build_tree_metadata([-1, 0, 1, 2], 16, 16)


def test_reference_signature_drop_in(fst, metadata_golden):
    case = metadata_golden["reftree_d7_bm128"]
    ai, am, li, bm, ma = unpack_golden_metadata(case)
    lin, lvl = orc.lineage_from_parent(case["parent"].tolist())
    lin_in = lin.clone()
    g_ai, g_am, g_li = fst.create_fst_attention_kernel_inputs(lin_in, lvl, block_m=bm, max_ancestors=ma)
    assert torch.equal(g_ai.cpu(), ai) and torch.equal(g_am.cpu(), am) and torch.equal(g_li.cpu(), li)
    # side effect of the reference (utils.py:124-125): each node written into its own row
    n = lin.shape[0]
    want = lin.clone()
    want[torch.arange(n), lvl] = torch.arange(n)
    assert torch.equal(lin_in, want)
    with pytest.raises(RuntimeError):
        fst.create_fst_attention_kernel_inputs(lin.clone(), lvl, block_m=bm, max_ancestors=8)


def test_out_buffers_are_reused(fst):
    from fstattention_b200 import configs
    meta = fst.build_tree_metadata(configs.random_window_tree(0), 64, 256)
    ptr = meta.packed.data_ptr()
    for s in (1, 2):
        par = configs.random_window_tree(s)
        fst.build_tree_metadata(par, 64, 256, out=meta)
        ai, am, li = orc.block_metadata_from_parent(par, 64, 256)
        assert meta.packed.data_ptr() == ptr
        assert torch.equal(meta.ancestor_idx.cpu(), ai) and torch.equal(meta.ancestor_mask.cpu(), am)
        assert torch.equal(meta.leaf_idx.cpu(), li)


def test_pack_kernel_round_trip(fst, metadata_golden):
    import ctypes
    from fstattention_b200 import _lib
    lib = _lib.lib()
    for name in ("medusa256_bm64", "random1024_s0_bm64", "binary31_bm16", "multiroot157_bm32"):
        case = metadata_golden[name]
        ai, am, li, bm, ma = unpack_golden_metadata(case)
        nb = ai.shape[0]
        for base in (0, 128):
            d_ai = (ai + base).cuda()            # sentinels shifted too, as the reference's test does
            d_li = (li + base).cuda()
            d_am = am.cuda()
            nbytes = lib.fst_packed_meta_bytes(nb, bm, ma)
            out = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            status = torch.zeros(4, dtype=torch.int32, device="cuda")
            rc = lib.fst_pack_metadata(d_ai.data_ptr(), d_am.data_ptr(), d_li.data_ptr(), 1, nb, bm, ma,
                                       base, out.data_ptr(), nbytes, status.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert status[0].item() == 0
            ref = fst.build_tree_metadata(case["parent"].tolist(), bm, ma).packed[0]
            got_parts = decode_packed(out.cpu().numpy(), nb, bm, ma)
            ref_parts = decode_packed(ref.cpu().numpy(), nb, bm, ma)
            for g, r in zip(got_parts, ref_parts):
                assert np.array_equal(g, r), (name, base)


def _reorder_cases():
    import random
    from fstattention_b200 import configs
    cases = {
        "single": [-1],
        "chain": [-1] + list(range(99)),
        "star": [-1] + [0] * 200,
        "forest_of_roots": [-1] * 40,
        "two_roots_interleaved": [-1, -1, 0, 1, 0, 1, 2, 3, 2, 3],
        "binary31": configs.binary_tree(),
        "medusa256": configs.workload("medusa256").trees[0],
        "random1024": configs.random_window_tree(3, 1024, 64),
        "wide_window": configs.random_window_tree(9, 700, 200),
        "deep4096": configs.workload("deep4096").trees[0],
    }
    rng = random.Random(5)
    cases["random8192"] = [-1] + [rng.randint(-1 if i % 97 == 0 else 0, i - 1) for i in range(1, 8192)]
    return cases


@pytest.mark.parametrize("name", list(_reorder_cases()))
def test_dfs_order_device_equals_host(fst, name):
    """The device renumbering is the host one, element for element."""
    par = _reorder_cases()[name]
    want_order, want_parent = fst.dfs_order(par)
    order, new_parent = fst.dfs_order_device(par)
    assert order.dtype == torch.int32 and order.is_cuda
    assert order.cpu().tolist() == want_order
    assert new_parent.cpu().tolist() == want_parent


def test_dfs_order_device_batch_and_errors(fst):
    from fstattention_b200 import configs
    trees = configs.workload("forest64").trees
    order, new_parent = fst.dfs_order_device(trees)
    assert order.shape == (64, 256)
    for t in (0, 17, 63):
        want_order, want_parent = fst.dfs_order(trees[t])
        assert order[t].cpu().tolist() == want_order and new_parent[t].cpu().tolist() == want_parent
    # the renumbered parents feed the precompute directly and need no more ancestors than before
    meta = fst.build_tree_metadata(new_parent, 64, 64)
    assert meta.check() is meta
    with pytest.raises(ValueError):
        fst.dfs_order_device([-1, 0, 5, 1])                  # parent after the node
    with pytest.raises(RuntimeError):
        fst.dfs_order_device([-1] + [0] * 8192)              # more nodes than the kernel holds



def test_reference_largest_context_131068_nodes(fst):
    """The largest tree of the reference's own tables (DEPTH_MAPPING[2**17] = 14, utils.py:4-13:
    131068 nodes), block 128, 64 ancestors: sampled blocks against the oracle, bit for bit."""
    lin, lvl = fst.create_tree(14)
    par = fst.parent_from_lineage(lin, lvl)
    n, bm, ma = par.shape[0], 128, 64
    assert n == 2 ** 17 - 4
    meta = fst.build_tree_metadata(par.to(torch.int32), bm, ma)
    nb = meta.n_blocks
    blocks = [0, 1, 2, 17, 255, 256, 511, nb // 2, nb - 2, nb - 1]
    ai, am, li = orc.block_metadata(lin, lvl, bm, ma, blocks=blocks)
    g_ai, g_am, g_li = (t.cpu() for t in meta)
    for b in blocks:
        assert torch.equal(g_ai[b], ai[b]), b
        assert torch.equal(g_am[b], am[b]), b
        assert torch.equal(g_li[b], li[b]), b
    # the documented node limit itself: segments of 4096 nodes whose first 64 are roots and whose
    # other nodes hang under one of them, so that ancestors sit at high node numbers
    n2 = 262144
    i = torch.arange(n2)
    par2 = torch.where(i % 4096 < 64, torch.full_like(i, -1), i // 4096 * 4096 + i % 64).to(torch.int32)
    meta2 = fst.build_tree_metadata(par2, 256, 128)
    cnt = meta2.packed.cpu().numpy()[0, : meta2.n_blocks * 4].view(np.int32)
    a2 = meta2.ancestor_idx.cpu()
    for b in (0, 1, 500, meta2.n_blocks - 1):
        lo = b * 256
        want = sorted({x for k in range(lo, lo + 256) for x in _ancestors(par2, k)})
        got = [int(x) for x in a2[b] if x >= 0]
        assert got == want, b
        assert cnt[b] == sum(1 for x in want if x < lo)


def _ancestors(par, k):
    out = []
    x = int(par[k])
    while x >= 0:
        out.append(x)
        x = int(par[x])
    return out


def test_size_that_does_not_fit_is_refused(fst):
    """block_m 1024 at the full node count needs more shared memory than an SM has: a clear
    status, not a launch failure."""
    from fstattention_b200 import _lib
    par = torch.full((262144,), -1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="beyond the supported limit"):
        fst.build_tree_metadata(par, 1024, 2048, reference_format=False)
    torch.cuda.synchronize()


def _topk_forest_cpu(scores, topk, lwf):
    """The construction build_tree_topk documents, with a stable sort on the CPU."""
    levels = scores.shape[0]
    parent, choice, cum = [-1] * topk, list(range(topk)), [list(map(float, scores[0]))]
    start = [0, topk]
    for l in range(1, levels):
        prev = np.array(cum[-1], dtype=np.float32)
        keep = int(len(prev) * lwf)
        order = np.argsort(-prev, kind="stable")[:keep]
        nxt = []
        for p in order:
            for k in range(topk):
                parent.append(start[l - 1] + int(p))
                choice.append(l * topk + k)
                nxt.append(np.float32(prev[p] + np.float32(scores[l, k])))
        cum.append(nxt)
        start.append(start[-1] + len(nxt))
    return parent, choice, [x for lvl in cum for x in lvl]


@pytest.mark.parametrize("depth,topk,lwf", [(7, 4, 0.5), (5, 10, 0.3), (9, 4, 0.5), (3, 3, 1.0)])
def test_device_built_tree_equals_create_tree_on_equal_scores(fst, depth, topk, lwf):
    lin, lvl = fst.create_tree(depth, topk, lwf)
    want = fst.parent_from_lineage(lin, lvl)
    scores = torch.zeros((depth + 1, topk), dtype=torch.float32, device="cuda")
    got = fst.build_tree_topk(scores, left_weight_factor=lwf)
    assert got.dtype == torch.int32 and got.shape == want.shape
    assert torch.equal(got.cpu().long(), want)
    assert fst.tree_topk_nodes(depth, topk, lwf) == want.shape[0]


def test_device_built_tree_follows_the_scores(fst):
    g = torch.Generator().manual_seed(8)
    depth, topk, lwf, T = 6, 4, 0.5, 5
    scores = torch.log_softmax(torch.randn((T, depth + 1, topk), generator=g), dim=-1)
    scores[1, 2] = scores[1, 2, 0]                       # a level of ties in one tree
    n = fst.tree_topk_nodes(depth, topk, lwf)
    parent, choice, nscore = fst.build_tree_topk(scores.cuda(), left_weight_factor=lwf, max_nodes=n + 12,
                                                 return_choice=True, return_scores=True)
    for t in range(T):
        wp, wc, ws = _topk_forest_cpu(scores[t].numpy(), topk, lwf)
        assert parent[t, :n].cpu().tolist() == wp, t
        assert choice[t, :n].cpu().tolist() == wc, t
        assert np.allclose(nscore[t, :n].cpu().numpy(), np.array(ws, dtype=np.float32), rtol=0, atol=1e-5)
        assert parent[t, n:].cpu().tolist() == [-1] * 12 and choice[t, n:].cpu().tolist() == [-1] * 12
    # cut by a node budget: the first max_nodes nodes of the same forest
    cut = fst.build_tree_topk(scores.cuda(), left_weight_factor=lwf, max_nodes=200)
    assert torch.equal(cut, parent[:, :200])
    # straight into the renumbering and the precompute, no host round trip
    order, new_parent = fst.dfs_order_device(parent[0, :n], check=False)
    meta = fst.build_tree_metadata(new_parent, 64, 64)
    want = orc.block_metadata_from_parent(new_parent.cpu().tolist(), 64, 64)
    for a, b in zip(meta, want):
        assert torch.equal(a.cpu(), b)
    with pytest.raises(ValueError, match="limits"):
        fst.tree_topk_nodes(14, 4, 0.5)                  # a level of 32768 nodes
