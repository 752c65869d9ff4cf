"""Tree attention kernels against the reference's outputs (golden) and the CPU oracle.

Tolerances.  fp16/bf16 kernels are gated at max-abs 2e-3 (fp16) against the oracle formula
evaluated on the same fp16 inputs in float32; against the oracle exactly as the reference
writes it (fp16 scores and probabilities) the gate is 2e-3 plus that formula's own measured
rounding error versus float64, because its noise alone exceeds 2e-3 at |out| ~ 4.  The
reference's own test accepts 1e-2 (fstattention.py:228).  fp32 inputs: 2e-5.
"""
import numpy as np
import pytest
import torch

from conftest import unpack_golden_metadata
from helpers import chain_mean_values, make_qkv, oracle_attention
from oracle import tree_oracle as orc

pytestmark = pytest.mark.gpu

TOL_F16 = 2e-3
TOL_BF16 = 1.6e-2          # bf16 has 8 fewer mantissa bits than fp16
TOL_F32 = 2e-5


@pytest.fixture(scope="module")
def fst(built_lib):
    import fstattention_b200
    return fstattention_b200


def kernels_for(dtype, d, bm, prefix=0):
    ks = ["auto", "simt"]
    if dtype in (torch.float16, torch.bfloat16) and d in (64, 128) and bm in (16, 32, 64, 128):
        ks += ["mma"] + (["tma_t32", "tma_t64"] if bm >= 32 else [])
        if bm in (64, 128) and prefix == 0:              # the persistent kernel: no shared prefix
            ks.append("persist")
    return ks


def maxabs(a, b):
    return (a.double() - b.double()).abs().max().item()


def test_golden_cases_all_kernels(fst, attention_golden):
    for name, case in attention_golden.items():
        q, k, v = (torch.from_numpy(case[x]) for x in ("q", "k", "v"))
        n, bm, ma, prefix = (int(case[x]) for x in ("n", "block_m", "max_ancestors", "prefix"))
        scale = float(case["sm_scale"])
        par = case["parent"].tolist()
        meta = fst.build_tree_metadata(par, bm, ma)
        dense = torch.from_numpy(case["out_dense"])[:, :, :n]
        tri = torch.from_numpy(case["out_triton"])[:, :, :n]
        exact32 = orc.tree_attention_reference(q, k, v, par, scale, bm, prefix, torch.float32)[:, :, :n]
        exact64 = orc.tree_attention_reference(q, k, v, par, scale, bm, prefix, torch.float64)[:, :, :n]
        noise = maxabs(dense, exact64)
        tol = TOL_F32 if q.dtype == torch.float32 else TOL_F16
        for kern in kernels_for(q.dtype, q.shape[-1], bm, prefix):
            o = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel=kern)
            o = o.cpu()[:, :, :n]
            assert torch.isfinite(o).all(), (name, kern)
            assert maxabs(o, exact32) <= tol, (name, kern, maxabs(o, exact32))
            assert maxabs(o, dense) <= tol + noise, (name, kern, maxabs(o, dense), noise)
            assert maxabs(o, tri) <= 1e-2, (name, kern)          # the reference test's own gate
        assert fst.last_status() == 0


def test_reference_call_sequence_with_prefix(fst, attention_golden):
    """The reference test's calling convention verbatim: tensors shifted by the prefix length,
    sentinels included (fstattention.py:211-212), then .to('cuda') and positional arguments."""
    case = attention_golden["reftree_d5_prefix128"]
    q, k, v = (torch.from_numpy(case[x]).cuda() for x in ("q", "k", "v"))
    n, bm, ma, prefix = (int(case[x]) for x in ("n", "block_m", "max_ancestors", "prefix"))
    ai, am, li = orc.block_metadata_from_parent(case["parent"].tolist(), bm, ma)
    ai += prefix
    li += prefix
    o = fst.fst_attention(q, k, v, ai.to("cuda"), am.to("cuda"), li.to("cuda"), float(case["sm_scale"]),
                          BLOCK_M=bm, MAX_ANCESTORS=ma)
    exact = orc.tree_attention_reference(q.cpu(), k.cpu(), v.cpu(), case["parent"].tolist(),
                                         float(case["sm_scale"]), bm, prefix, torch.float32)
    assert maxabs(o.cpu()[:, :, :n], exact[:, :, :n]) <= TOL_F16
    # and with this package's own precompute, shifted in place the same way
    g_ai, g_am, g_li = fst.build_tree_metadata(case["parent"].tolist(), bm, ma)
    g_ai += prefix
    g_li += prefix
    o2 = fst.fst_attention(q, k, v, g_ai, g_am, g_li, float(case["sm_scale"]), BLOCK_M=bm, MAX_ANCESTORS=ma)
    assert torch.equal(o, o2)
    assert fst.last_status() == 0


WORKLOAD_CASES = [("binary31", 4, None), ("medusa256", 32, None), ("random1024", 8, 0),
                  ("random1024", 4, 7), ("deep4096", 2, None)]


@pytest.mark.parametrize("name,heads,step", WORKLOAD_CASES)
def test_workloads_vs_oracle(fst, name, heads, step):
    from fstattention_b200 import configs
    w = configs.workload(name, step or 0)
    dtype = {"fp16": torch.float16, "fp32": torch.float32}[w.dtype]
    par = w.trees[0]
    n = len(par)
    q, k, v = make_qkv(1, heads, n, n, w.head_dim, dtype, seed=11)
    meta = fst.build_tree_metadata(par, w.block_m, w.max_ancestors)
    exact = oracle_attention(q, k, v, par, w.sm_scale, compute_dtype=torch.float32, head_chunk=2)
    tol = TOL_F32 if dtype == torch.float32 else TOL_F16
    for kern in kernels_for(dtype, w.head_dim, w.block_m):
        o = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=w.sm_scale, kernel=kern).cpu()
        assert maxabs(o, exact) <= tol, (name, kern, maxabs(o, exact))
    assert fst.last_status() == 0


def test_forest_per_tree_metadata(fst):
    from fstattention_b200 import configs
    w = configs.workload("forest64")
    trees = w.trees[:8]
    q, k, v = make_qkv(8, 4, 256, 256, 128, torch.float16, seed=5)
    meta = fst.build_tree_metadata(trees, w.block_m, w.max_ancestors)
    o = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=w.sm_scale).cpu()
    for t in range(8):
        exact = oracle_attention(q[t:t + 1], k[t:t + 1], v[t:t + 1], trees[t], w.sm_scale,
                                 compute_dtype=torch.float32)
        assert maxabs(o[t:t + 1], exact) <= TOL_F16, t
    # reference-format tensors with a leading tree dimension give the same answer
    ai, am, li = meta
    ai2, am2, li2 = ai.clone(), am.clone(), li.clone()
    o2 = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), ai2, am2, li2, w.sm_scale,
                           BLOCK_M=w.block_m, MAX_ANCESTORS=w.max_ancestors).cpu()
    assert torch.equal(o, o2)


@pytest.mark.parametrize("name", ["medusa256", "random1024", "forest64", "deep4096"])
def test_full_size_equal_scores_property(fst, name):
    """Full BASELINE sizes.  With K = 0 every attended key gets the same weight, so each output
    row must be the mean of V over the node and its ancestors - computable exactly in O(N)."""
    from fstattention_b200 import configs
    w = configs.workload(name)
    T, n, H, D = len(w.trees), w.n_nodes, w.heads, w.head_dim
    g = torch.Generator().manual_seed(3)
    v = torch.randn((T, H, n, D), generator=g).half()
    q = torch.randn((T, H, n, D), generator=g).half()
    k = torch.zeros_like(v)
    meta = fst.build_tree_metadata(w.trees if T > 1 else w.trees[0], w.block_m, w.max_ancestors)
    for kern in ("mma", "tma_t32", "tma_t64", "persist"):
        o = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=w.sm_scale, kernel=kern).cpu()
        for t in range(0, T, 9):
            want = chain_mean_values(w.trees[t], v[t].double().numpy())
            err = np.abs(o[t].double().numpy() - want).max()
            assert err <= TOL_F16, (name, kern, t, err)
    # rows sum to one: V = 1 gives exactly 1 whatever the scores are
    k = torch.randn((T, H, n, D), generator=g).half()
    o = fst.fst_attention(q.cuda(), k.cuda(), torch.ones_like(v).cuda(), meta, sm_scale=w.sm_scale).cpu()
    assert (o.float() - 1).abs().max().item() <= 1e-3
    assert fst.last_status() == 0


def test_full_size_kernels_agree(fst):
    """deep4096 at full head count: tensor-core kernels against the fp32 SIMT kernel."""
    from fstattention_b200 import configs
    w = configs.workload("deep4096")
    q, k, v = (x.cuda() for x in make_qkv(1, w.heads, w.n_nodes, w.n_nodes, w.head_dim, torch.float16, 17))
    meta = fst.build_tree_metadata(w.trees[0], w.block_m, w.max_ancestors)
    base = fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, kernel="simt")
    for kern in ("mma", "tma_t32", "tma_t64", "persist"):
        o = fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, kernel=kern)
        assert maxabs(o, base) <= TOL_F16, kern


@pytest.mark.parametrize("dtype,d,bm,prefix", [
    (torch.float16, 128, 64, 64), (torch.float16, 128, 64, 200), (torch.float16, 64, 128, 37),
    (torch.bfloat16, 128, 64, 0), (torch.bfloat16, 64, 32, 96), (torch.float16, 32, 64, 16),
    (torch.float32, 16, 16, 5), (torch.float32, 128, 128, 130), (torch.float16, 128, 16, 0),
])
def test_shapes_dtypes_and_prefix(fst, dtype, d, bm, prefix):
    from fstattention_b200 import configs
    par = configs.random_window_tree(5, 300, 24)        # 300 rows: partial last block
    n = len(par)
    q, k, v = make_qkv(2, 3, n, prefix + n, d, dtype, seed=9)
    ma = 128
    meta = fst.build_tree_metadata(par, bm, ma)
    scale = d ** -0.5
    exact = oracle_attention(q, k, v, par, scale, prefix=prefix, compute_dtype=torch.float32)
    tol = {torch.float16: TOL_F16, torch.bfloat16: TOL_BF16, torch.float32: TOL_F32}[dtype]
    for kern in kernels_for(dtype, d, bm, prefix):
        o, lse = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel=kern,
                                   return_lse=True)
        assert maxabs(o.cpu(), exact) <= tol, (kern, maxabs(o.cpu(), exact))
        # base-2 log-sum-exp of the scaled scores (fstattention.py:140-141)
        lin, _ = orc.lineage_from_parent(par)
        mask = torch.cat((torch.ones((n, prefix)), orc.full_attention_mask(lin, 0)), dim=1)
        s = torch.matmul(q.double(), k.double().transpose(2, 3)) * scale
        s[:, :, mask == 0] = float("-inf")
        want = torch.logsumexp(s, dim=-1) / np.log(2.0)
        assert maxabs(lse.cpu().view(2, 3, n), want) <= (2e-2 if dtype == torch.bfloat16 else 2e-3), kern
    assert fst.last_status() == 0


def test_strided_inputs_and_out_argument(fst):
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, D = 256, 4, 128
    g = torch.Generator().manual_seed(2)
    # [Z, N, H, D] storage viewed as [Z, H, N, D], as a projection layer would leave it
    q, k, v = (torch.randn((2, n, H, D), generator=g).half().cuda().permute(0, 2, 1, 3) for _ in range(3))
    meta = fst.build_tree_metadata(par, 64, 64)
    out = torch.empty((2, n, H, D), dtype=torch.float16, device="cuda").permute(0, 2, 1, 3)
    o = fst.fst_attention(q, k, v, meta, sm_scale=D ** -0.5, out=out)
    assert o.data_ptr() == out.data_ptr()
    exact = oracle_attention(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), par,
                             D ** -0.5, compute_dtype=torch.float32)
    assert maxabs(o.cpu(), exact) <= TOL_F16


def test_padded_tensors_phantom_rows(fst):
    """Tensors padded to a whole number of blocks, as the reference pads 2^k-4 trees to 2^k:
    rows past the last node attend only to themselves and the real rows are unaffected."""
    par = [-1] + [(i - 1) // 2 for i in range(1, 31)]
    q, k, v = make_qkv(1, 2, 32, 32, 64, torch.float16, seed=4)
    meta = fst.build_tree_metadata(par, 16, 16)
    o = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=0.125).cpu()
    exact = oracle_attention(q[:, :, :31], k[:, :, :31], v[:, :, :31], par, 0.125, compute_dtype=torch.float32)
    assert maxabs(o[:, :, :31], exact) <= TOL_F16
    assert maxabs(o[:, :, 31], v[:, :, 31]) <= 1e-3


def test_argument_errors_are_python_errors(fst):
    par = [-1, 0, 0, 1]
    meta = fst.build_tree_metadata(par, 16, 16)
    q = torch.randn(1, 1, 4, 64).half()
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        fst.fst_attention(q, q, q, meta, sm_scale=1.0)
    qc = q.cuda()
    with pytest.raises(AssertionError):
        fst.fst_attention(qc[..., :24], qc[..., :24], qc[..., :24], meta, sm_scale=1.0)
    with pytest.raises(RuntimeError, match="unsupported"):
        fst.fst_attention(qc.float(), qc.float(), qc.float(), meta, sm_scale=1.0, kernel="mma")
    odd = torch.randn(1, 1, 4, 72).half().cuda()[..., 4:68]           # rows start 8 bytes off
    with pytest.raises(RuntimeError, match="aligned"):
        fst.fst_attention(odd, odd, odd, meta, sm_scale=1.0, kernel="mma")
    fst.fst_attention(odd, odd, odd, meta, sm_scale=1.0, kernel="simt")   # the SIMT kernel takes it
    torch.cuda.synchronize()


@pytest.mark.parametrize("shared_kv_prefix", [True, False])
def test_reference_test_op_recipe(fst, shared_kv_prefix):
    """The reference's own test, step for step (fstattention.py:183-228), with this package
    behind the reference's names: Z=2, H=2, N_CTX=2048, D=64, fp16, seed 20, std 0.5, scale 0.5,
    BLOCK_M=128, MAX_ANCESTORS=64, atol 1e-2 on all rows but the four pad rows."""
    Z, H, N_CTX, D_HEAD, dtype = 2, 2, 2 ** 11, 64, torch.float16
    torch.manual_seed(20)
    q = torch.empty((Z, H, N_CTX, D_HEAD), dtype=dtype, device="cuda").normal_(mean=0.0, std=0.5)
    kv_rows = 2 * N_CTX if shared_kv_prefix else N_CTX
    k = torch.empty((Z, H, kv_rows, D_HEAD), dtype=dtype, device="cuda").normal_(mean=0.0, std=0.5)
    v = torch.empty((Z, H, kv_rows, D_HEAD), dtype=dtype, device="cuda").normal_(mean=0.0, std=0.5)
    sm_scale = 0.5

    lineage, level_lookup = fst.create_tree(depth=fst.DEPTH_MAPPING[N_CTX])
    full_mask = fst.create_full_attention_mask(lineage)
    BLOCK_M = 128
    MAX_ANCESTORS = fst.MAX_ANCESTOR_MAPPING[N_CTX]
    ancestor_idx, ancestor_mask, leaf_idx = fst.create_fst_attention_kernel_inputs(
        lineage, level_lookup, block_m=BLOCK_M, max_ancestors=MAX_ANCESTORS)
    if shared_kv_prefix:
        full_mask = torch.cat((torch.ones((N_CTX, N_CTX), dtype=torch.bool), full_mask), dim=1)
        ancestor_idx += N_CTX
        leaf_idx += N_CTX

    M = full_mask.to("cuda")
    p = torch.matmul(q, k.transpose(2, 3)) * sm_scale
    p[:, :, M == 0] = float("-inf")
    p = torch.softmax(p.float(), dim=-1).half()
    ref_out = torch.matmul(p, v)

    ancestor_idx, ancestor_mask, leaf_idx = ancestor_idx.to("cuda"), ancestor_mask.to("cuda"), leaf_idx.to("cuda")
    out = fst.fst_attention(q, k, v, ancestor_idx, ancestor_mask, leaf_idx, sm_scale).half()
    assert torch.allclose(ref_out[:, :, :-4], out[:, :, :-4], atol=1e-2, rtol=0)
    assert fst.last_status() == 0


@pytest.mark.parametrize("prefix,splits", [(1000, 3), (4096, 8), (130, 2), (64, 5)])
def test_prefix_split_over_ctas(fst, prefix, splits):
    """A shared prefix cut into runs handled by separate CTAs and merged afterwards gives the
    same output and log-sum-exp as the single-pass kernel and as the oracle."""
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, D = 256, 3, 128
    q, k, v = make_qkv(2, H, n, prefix + n, D, torch.float16, seed=21)
    meta = fst.build_tree_metadata(par, 64, 64)
    scale = D ** -0.5
    exact = oracle_attention(q, k, v, par, scale, prefix=prefix, compute_dtype=torch.float32)
    one, lse_one = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kv_splits=1, return_lse=True)
    for kern in ("tma_t32", "tma_t64", "tma_umma", "auto"):
        out, lse = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kv_splits=splits,
                                     return_lse=True, kernel=kern)
        assert maxabs(out.cpu(), exact) <= TOL_F16, (kern, maxabs(out.cpu(), exact))
        assert maxabs(out, one) <= TOL_F16
        assert maxabs(lse, lse_one) <= 2e-3
    auto = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale)       # automatic split
    assert maxabs(auto.cpu(), exact) <= TOL_F16
    assert fst.last_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefix_with_head_dim_64(fst, dtype):
    """head_dim 64: the tcgen05 prefix kernel (64-column Q / K / V tiles), the tree kernel walking
    the prefix alone or split over CTAs, and the automatic choice."""
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, D, prefix = 256, 3, 64, 900
    q, k, v = make_qkv(2, H, n, prefix + n, D, dtype, seed=81)
    scale = D ** -0.5
    exact = oracle_attention(q, k, v, par, scale, prefix=prefix, compute_dtype=torch.float32)
    meta = fst.build_tree_metadata(par, 64, 64)
    tol = TOL_F16 if dtype == torch.float16 else TOL_BF16
    for kern, splits in (("auto", None), ("auto", 4), ("tma_umma", 1), ("tma_umma", 3), ("tma_t32", 3),
                         ("tma_t64", 1), ("mma", None), ("simt", None)):
        out = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel=kern, kv_splits=splits)
        assert maxabs(out.cpu(), exact) <= tol, (kern, splits, maxabs(out.cpu(), exact))
    assert fst.last_status() == 0


@pytest.mark.parametrize("prefix,runs,n,dtype", [(128, 1, 256, torch.float16), (129, 2, 200, torch.float16),
                                                  (700, 1, 256, torch.float16), (1111, 3, 130, torch.float16),
                                                  (1111, 2, 256, torch.bfloat16)])
def test_prefix_tcgen05_moving_maximum(fst, prefix, runs, n, dtype):
    """The tcgen05 prefix kernel with scores that keep growing along the prefix, so that the
    reference point of its exponentials has to move (and the accumulator in tensor memory be
    rescaled) several times; odd and single tile counts, ragged last tiles, ragged query rows."""
    from fstattention_b200 import configs
    par = configs.random_window_tree(5, n, 40)
    H, D = 2, 128
    q, k, v = make_qkv(1, H, n, prefix + n, D, dtype, seed=41)
    ramp = torch.linspace(0.0, 4.0, prefix).view(1, 1, prefix, 1)
    k[:, :, :prefix] = (k[:, :, :prefix].float() * 0.05 + ramp).to(dtype)      # q.k grows by ~250 along the prefix
    q = (q.float() * 0.05 + 0.5).to(dtype)
    scale = D ** -0.5
    exact = oracle_attention(q, k, v, par, scale, prefix=prefix, compute_dtype=torch.float32)
    meta = fst.build_tree_metadata(par, 64, 128)
    out, lse = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel="tma_umma",
                                 kv_splits=runs, return_lse=True)
    tol = TOL_F16 if dtype == torch.float16 else TOL_BF16
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    assert maxabs(out.cpu(), exact) <= tol, maxabs(out.cpu(), exact)
    one, lse_one = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel="tma_t64",
                                     kv_splits=1, return_lse=True)
    assert maxabs(lse, lse_one) <= (2e-3 if dtype == torch.float16 else 2e-2)
    assert fst.last_status() == 0


def test_prefix_tcgen05_in_a_cuda_graph(fst):
    """The prefix path forks its tree kernel onto a second stream; captured into a CUDA graph and
    replayed on new data it gives what the eager call gives."""
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, D, prefix = 256, 4, 128, 1024
    meta = fst.build_tree_metadata(par, 64, 64)
    scale = D ** -0.5
    q, k, v = (t.cuda() for t in make_qkv(1, H, n, prefix + n, D, torch.float16, seed=51))
    out = torch.empty_like(q)
    fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_umma", kv_splits=2, out=out)   # warm-up, eager
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_umma", kv_splits=2, out=out)
    q2, k2, v2 = (t.cuda() for t in make_qkv(1, H, n, prefix + n, D, torch.float16, seed=52))
    q.copy_(q2); k.copy_(k2); v.copy_(v2)
    graph.replay()
    torch.cuda.synchronize()
    eager = fst.fst_attention(q2, k2, v2, meta, sm_scale=scale, kernel="tma_umma", kv_splits=2)
    assert maxabs(out, eager) == 0.0
    exact = oracle_attention(q2.cpu(), k2.cpu(), v2.cpu(), par, scale, prefix=prefix, compute_dtype=torch.float32)
    assert maxabs(out.cpu(), exact) <= TOL_F16
    assert fst.last_status() == 0


@pytest.mark.parametrize("prefix", [0, 512])
def test_grouped_query_attention(fst, prefix):
    """K and V with fewer heads than Q: query head h reads K/V head h // (H / H_kv).  Checked
    against the oracle on K/V with the heads repeated, for every kernel, with and without a
    shared prefix (where the tcgen05 prefix kernel and the split tree kernel take part)."""
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, H_kv, D = 256, 8, 2, 128
    q, _, _ = make_qkv(2, H, n, prefix + n, D, torch.float16, seed=61)
    _, k, v = make_qkv(2, H_kv, n, prefix + n, D, torch.float16, seed=62)
    scale = D ** -0.5
    k_rep, v_rep = (t.repeat_interleave(H // H_kv, dim=1) for t in (k, v))
    exact = oracle_attention(q, k_rep, v_rep, par, scale, prefix=prefix, compute_dtype=torch.float32)
    meta = fst.build_tree_metadata(par, 64, 64)
    kernels = ["auto", "simt", "mma", "tma_t32", "tma_t64"] + (["tma_umma"] if prefix else [])
    for kern in kernels:
        for splits in ((1, 2) if prefix and kern not in ("simt", "mma") else (None,)):
            out, lse = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel=kern,
                                         kv_splits=splits, return_lse=True)
            assert maxabs(out.cpu(), exact) <= TOL_F16, (kern, splits, maxabs(out.cpu(), exact))
            same = fst.fst_attention(q.cuda(), k_rep.cuda(), v_rep.cuda(), meta, sm_scale=scale, kernel=kern,
                                     kv_splits=splits)
            assert torch.equal(out, same), (kern, splits)      # the same arithmetic on the same rows
    with pytest.raises(ValueError):
        fst.fst_attention(q.cuda(), k[:, :1].repeat(1, 3, 1, 1).cuda(), v[:, :1].repeat(1, 3, 1, 1).cuda(), meta,
                          sm_scale=scale)                       # 8 query heads over 3 K/V heads
    assert fst.last_status() == 0


def _scatter_into_pages(k, v, prefix_lens, page_size, layout, seed):
    """Put the prefix rows of [Z, H_kv, P_max + N, D] tensors into a shuffled page pool."""
    Z, H_kv, _, D = k.shape
    pages_per_seq = [-(-p // page_size) for p in prefix_lens]
    n_pages = sum(pages_per_seq) + 3                      # a few pages nobody owns
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    shape = (n_pages, page_size, H_kv, D) if layout == "NHD" else (n_pages, H_kv, page_size, D)
    k_pool = torch.randn(shape, generator=g).to(k.dtype)  # unowned rows hold finite junk
    v_pool = torch.randn(shape, generator=g).to(k.dtype)
    table = torch.full((Z, max(pages_per_seq) + 1), -7, dtype=torch.int32)   # entries past a sequence are junk
    nxt = 0
    for z in range(Z):
        for i in range(pages_per_seq[z]):
            pid = perm[nxt]; nxt += 1
            table[z, i] = pid
            rows = min(page_size, prefix_lens[z] - i * page_size)
            src = slice(i * page_size, i * page_size + rows)
            if layout == "NHD":
                k_pool[pid, :rows] = k[z, :, src].transpose(0, 1)
                v_pool[pid, :rows] = v[z, :, src].transpose(0, 1)
            else:
                k_pool[pid, :, :rows] = k[z, :, src]
                v_pool[pid, :, :rows] = v[z, :, src]
    return k_pool, v_pool, table


@pytest.mark.parametrize("page_size,layout,dtype,D", [(16, "NHD", torch.float16, 128), (64, "HND", torch.float16, 128),
                                                     (128, "NHD", torch.bfloat16, 128), (32, "NHD", torch.float16, 128),
                                                     (16, "HND", torch.float16, 64)])
def test_paged_prefix(fst, page_size, layout, dtype, D):
    """Prefix rows in a shuffled page pool with a different length per batch element, tree rows
    in their own tensors, grouped K/V heads: equal to attention over the same rows laid out
    contiguously (oracle), and to the contiguous tcgen05 path where the lengths allow."""
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, H_kv = 256, 4, 2
    prefix_lens = [700, 129, 1024]
    Z, p_max = len(prefix_lens), max(prefix_lens)
    q, _, _ = make_qkv(Z, H, n, n, D, dtype, seed=71)
    _, k, v = make_qkv(Z, H_kv, n, p_max + n, D, dtype, seed=72)     # rows [0, P_z) prefix, [p_max, p_max + n) tree
    scale = D ** -0.5
    meta = fst.build_tree_metadata(par, 64, 64)
    k_pool, v_pool, table = _scatter_into_pages(k, v, prefix_lens, page_size, layout, seed=73)
    k_tree, v_tree = k[:, :, p_max:].contiguous(), v[:, :, p_max:].contiguous()
    lens = torch.tensor(prefix_lens, dtype=torch.int32)
    tol = TOL_F16 if dtype == torch.float16 else TOL_BF16
    for splits in (1, 3, None):
        out, lse = fst.fst_attention_paged(q.cuda(), k_tree.cuda(), v_tree.cuda(), meta, k_pool.cuda(), v_pool.cuda(),
                                           table.cuda(), lens.cuda(), scale, pool_layout=layout, kv_splits=splits,
                                           return_lse=True)
        assert torch.isfinite(out).all()
        for z, pz in enumerate(prefix_lens):
            kz = torch.cat([k[z:z + 1, :, :pz], k[z:z + 1, :, p_max:]], dim=2).repeat_interleave(H // H_kv, dim=1)
            vz = torch.cat([v[z:z + 1, :, :pz], v[z:z + 1, :, p_max:]], dim=2).repeat_interleave(H // H_kv, dim=1)
            exact = oracle_attention(q[z:z + 1], kz, vz, par, scale, prefix=pz, compute_dtype=torch.float32)
            assert maxabs(out[z:z + 1].cpu(), exact) <= tol, (splits, z, maxabs(out[z:z + 1].cpu(), exact))
    # the longest sequence against the contiguous path with the same number of runs: same tiles, same bits
    z = prefix_lens.index(p_max)
    cont = fst.fst_attention(q[z:z + 1].cuda(), k[z:z + 1].cuda(), v[z:z + 1].cuda(), meta, sm_scale=scale,
                             kernel="tma_umma", kv_splits=3)
    paged = fst.fst_attention_paged(q[z:z + 1].cuda(), k_tree[z:z + 1].cuda(), v_tree[z:z + 1].cuda(), meta,
                                    k_pool.cuda(), v_pool.cuda(), table[z:z + 1].contiguous().cuda(), lens[z:z + 1].cuda(),
                                    scale, pool_layout=layout, kv_splits=3)
    assert torch.equal(cont, paged)
    assert fst.last_status() == 0


def test_paged_prefix_with_an_empty_sequence(fst):
    """One batch element has no prefix at all (and junk in its block-table row): it gets plain
    tree attention while its neighbours get theirs behind their prefixes."""
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, D, page_size = 256, 2, 128, 32
    prefix_lens = [300, 0, 65]
    Z, p_max = len(prefix_lens), max(prefix_lens)
    q, _, _ = make_qkv(Z, H, n, n, D, torch.float16, seed=91)
    _, k, v = make_qkv(Z, H, n, p_max + n, D, torch.float16, seed=92)
    scale = D ** -0.5
    meta = fst.build_tree_metadata(par, 64, 64)
    k_pool, v_pool, table = _scatter_into_pages(k, v, prefix_lens, page_size, "NHD", seed=93)
    k_tree, v_tree = k[:, :, p_max:].contiguous(), v[:, :, p_max:].contiguous()
    lens = torch.tensor(prefix_lens, dtype=torch.int32)
    out, lse = fst.fst_attention_paged(q.cuda(), k_tree.cuda(), v_tree.cuda(), meta, k_pool.cuda(), v_pool.cuda(),
                                       table.cuda(), lens.cuda(), scale, kv_splits=2, return_lse=True)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    for z, pz in enumerate(prefix_lens):
        kz = torch.cat([k[z:z + 1, :, :pz], k[z:z + 1, :, p_max:]], dim=2)
        vz = torch.cat([v[z:z + 1, :, :pz], v[z:z + 1, :, p_max:]], dim=2)
        exact = oracle_attention(q[z:z + 1], kz, vz, par, scale, prefix=pz, compute_dtype=torch.float32)
        assert maxabs(out[z:z + 1].cpu(), exact) <= TOL_F16, (z, maxabs(out[z:z + 1].cpu(), exact))
    assert fst.last_status() == 0


def test_prefix_path_from_two_threads_on_their_own_streams(fst):
    """The forked prefix path keeps its helper stream per host thread: two threads, each on its
    own stream, calling it at the same time get what a single call gets."""
    import threading
    from fstattention_b200 import configs
    par = configs.left_weighted_tree()
    n, H, D, prefix = 256, 4, 128, 1024
    meta = fst.build_tree_metadata(par, 64, 64)
    scale = D ** -0.5
    data = [tuple(t.cuda() for t in make_qkv(1, H, n, prefix + n, D, torch.float16, seed=100 + i)) for i in range(2)]
    want = [fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_umma", kv_splits=2) for q, k, v in data]
    torch.cuda.synchronize()
    got = [None, None]
    errors = []

    def worker(i):
        try:
            stream = torch.cuda.Stream()
            q, k, v = data[i]
            with torch.cuda.stream(stream):
                for _ in range(20):
                    out = fst.fst_attention(q, k, v, meta, sm_scale=scale, kernel="tma_umma", kv_splits=2)
            stream.synchronize()
            got[i] = out
        except Exception as exc:                          # surfaced in the main thread below
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    for i in range(2):
        assert torch.equal(got[i], want[i]), i
    assert fst.last_status() == 0


def test_a_wait_that_nobody_answers_runs_out(fst):
    """The time limit on mbarrier waits: a kernel waiting on a barrier nobody arrives at gives
    up, reports FST_DEV_TIMEOUT and ends; the context is fine afterwards."""
    import time
    from fstattention_b200 import _lib
    lib = _lib.lib()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = lib.fst_selftest_wait_timeout(status.data_ptr(), done.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert status[:2].tolist() == [19, 12345] and done.item() == 2
    assert 0.03 <= took <= 2.0, took
    assert "wait" in _lib.status_string(19)
    x = torch.ones(1024, device="cuda")                      # the device still answers
    assert x.sum().item() == 1024.0


def test_dfs_renumbering_leaves_the_result_unchanged(fst):
    """Attention on the depth-first renumbered tree, rows permuted in and scattered back, equals
    attention on the original numbering (and the oracle), while gathering fewer rows."""
    from fstattention_b200 import configs
    par = configs.random_window_tree(9, 700, 200)       # wide window: ancestors far away in index space
    n, H, D = len(par), 2, 128
    q, k, v = make_qkv(1, H, n, n, D, torch.float16, seed=31)
    scale = D ** -0.5
    exact = oracle_attention(q, k, v, par, scale, compute_dtype=torch.float32)
    order, new_par = fst.dfs_order(par)
    idx = torch.tensor(order)
    meta = fst.build_tree_metadata(new_par, 64, 512)
    o_perm = fst.fst_attention(q[:, :, idx].cuda(), k[:, :, idx].cuda(), v[:, :, idx].cuda(), meta, sm_scale=scale)
    out = torch.empty_like(o_perm)
    out[:, :, idx.cuda()] = o_perm
    assert maxabs(out.cpu(), exact) <= TOL_F16
    before = fst.build_tree_metadata(par, 64, 700)
    assert int(meta.packed.view(torch.int32)[0, :meta.n_blocks].sum()) < int(before.packed.view(torch.int32)[0, :before.n_blocks].sum())


@pytest.mark.parametrize("scale", [-0.3, 0.0, -1.0 / 128 ** 0.5])
def test_any_finite_scale_as_the_reference(fst, scale):
    """The reference scales the scores before the row maximum (fstattention.py:78-97) and so takes
    a factor of either sign; every kernel here must give the oracle's answer for it too, also
    behind a prefix long enough for the split paths."""
    from fstattention_b200 import configs
    par = configs.random_window_tree(3, 200, 16)
    n = len(par)
    for dtype, d, bm, prefix in ((torch.float16, 128, 64, 0), (torch.float16, 64, 32, 300), (torch.float32, 32, 16, 7)):
        q, k, v = make_qkv(1, 2, n, prefix + n, d, dtype, seed=21)
        meta = fst.build_tree_metadata(par, bm, 128)
        exact = oracle_attention(q, k, v, par, scale, prefix=prefix, compute_dtype=torch.float32)
        tol = TOL_F32 if dtype == torch.float32 else TOL_F16
        for kern in kernels_for(dtype, d, bm, prefix):
            o, lse = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=scale, kernel=kern,
                                       return_lse=True)
            assert maxabs(o.cpu(), exact) <= tol, (scale, dtype, kern, maxabs(o.cpu(), exact))
            assert torch.isfinite(lse).all()
    q = torch.zeros((1, 1, n, 64), dtype=torch.float16, device="cuda")
    for bad in (float("nan"), float("inf")):
        with pytest.raises(ValueError, match="finite"):
            fst.fst_attention(q, q, q, meta, sm_scale=bad)
    # the C entry point refuses it as well
    from fstattention_b200 import _lib
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = _lib.lib().fst_attention_fwd(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), None,
                                      meta.packed.data_ptr(), 0, 1, 1, n, n, 64, *q.stride()[:3], *q.stride()[:3],
                                      *q.stride()[:3], *q.stride()[:3], 16, 128, float("nan"), 0, 0, st.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    assert fst.last_status() == 0


def test_status_record_can_be_cleared(fst):
    """One recorded problem must not stick for the life of the process."""
    par = [-1, 0, 0, 1]
    meta = fst.build_tree_metadata(par, 16, 16)
    q = torch.randn(1, 1, 4, 64).half().cuda()
    fst.fst_attention(q, q, q, meta, sm_scale=1.0)
    assert fst.last_status() == 0
    # metadata that points past the K/V rows: recorded, not a fault
    ai, am, li = (t.clone() for t in meta)
    ai[0, 0] = 99
    am[0, 3, 0] = True
    fst.fst_attention(q, q, q, ai, am, li, 1.0, BLOCK_M=16, MAX_ANCESTORS=16)
    assert fst.last_status() == 18                      # FST_DEV_INDEX_RANGE
    assert fst.last_status(clear=True) == 18
    assert fst.last_status() == 0
    fst.fst_attention(q, q, q, ai, am, li, 1.0, BLOCK_M=16, MAX_ANCESTORS=16)
    assert fst.last_status() == 18
    fst.clear_status()
    o = fst.fst_attention(q, q, q, meta, sm_scale=1.0)
    assert fst.last_status() == 0 and torch.isfinite(o).all()


def test_metadata_fetched_ahead_of_the_dependency_wait(fst):
    """From the second call after a precompute on, the Python layer lets the kernel read its index
    lists before it waits for the launch ahead of it.  Results must not depend on that: a run of
    back-to-back layers, eagerly and as a replayed CUDA graph with the tree changing between
    replays, against calls that each follow their own precompute."""
    from fstattention_b200 import configs, _lib
    trees = [configs.random_window_tree(s, 512, 48) for s in range(4)]
    H, D, n = 8, 128, 512
    layers = [tuple(x.cuda() for x in make_qkv(1, H, n, n, D, torch.float16, seed=40 + i)) for i in range(6)]
    parent = torch.tensor(trees[0], dtype=torch.int32, device="cuda")
    meta = fst.build_tree_metadata(parent, 64, 320, reference_format=False)
    outs = [torch.empty_like(l[0]) for l in layers]

    def step():
        fst.build_tree_metadata(parent, 64, 320, out=meta, check=False)
        for (q, k, v), o in zip(layers, outs):
            fst.fst_attention(q, k, v, meta, sm_scale=D ** -0.5, out=o)

    step()
    assert meta.reads_since_build == len(layers)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for t, par in enumerate(trees):
        parent.copy_(torch.tensor(par, dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        fresh = fst.build_tree_metadata(par, 64, 320, reference_format=False)
        for (q, k, v), o in zip(layers, outs):
            fresh.reads_since_build = 0                   # every call as the first after its precompute
            want = fst.fst_attention(q, k, v, fresh, sm_scale=D ** -0.5)
            assert torch.equal(o, want), t
    exact = oracle_attention(*(x.cpu() for x in layers[-1]), trees[-1], D ** -0.5, compute_dtype=torch.float32, head_chunk=2)
    assert maxabs(outs[-1].cpu(), exact) <= TOL_F16
    assert fst.last_status() == 0


def test_forest64_full_size_against_the_oracle(fst):
    """All 64 trees x 32 heads of the batched configuration, dense oracle tree by tree."""
    from fstattention_b200 import configs
    w = configs.workload("forest64")
    T, H, n, D = len(w.trees), w.heads, w.n_nodes, w.head_dim
    q, k, v = make_qkv(T, H, n, n, D, torch.float16, seed=61)
    meta = fst.build_tree_metadata(w.trees, w.block_m, w.max_ancestors, reference_format=False)
    outs = {kern: fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=w.sm_scale, kernel=kern).cpu()
            for kern in ("auto", "tma_t32", "persist")}
    worst = dict.fromkeys(outs, 0.0)
    for t in range(T):
        exact = oracle_attention(q[t:t + 1], k[t:t + 1], v[t:t + 1], w.trees[t], w.sm_scale,
                                 compute_dtype=torch.float32)
        for kern, o in outs.items():
            worst[kern] = max(worst[kern], maxabs(o[t:t + 1], exact))
    assert max(worst.values()) <= TOL_F16, worst
    assert fst.last_status() == 0


def test_deep4096_all_heads_row_slices_against_the_oracle(fst):
    """The deep tree at its full head count: every head, the query rows of the first, a middle and
    the last two blocks against the dense oracle."""
    from fstattention_b200 import configs
    w = configs.workload("deep4096")
    H, n, D = w.heads, w.n_nodes, w.head_dim
    q, k, v = make_qkv(1, H, n, n, D, torch.float16, seed=62)
    meta = fst.build_tree_metadata(w.trees[0], w.block_m, w.max_ancestors, reference_format=False)
    lin, _ = orc.lineage_from_parent(w.trees[0])
    mask = orc.full_attention_mask(lin, pad_rows=0)
    rows = torch.cat([torch.arange(0, 64), torch.arange(2048, 2112), torch.arange(n - 128, n)])
    exact = orc.dense_tree_attention(q[:, :, rows], k, v, mask[rows], w.sm_scale, torch.float32, head_chunk=8)
    for kern in ("auto", "persist"):
        o = fst.fst_attention(q.cuda(), k.cuda(), v.cuda(), meta, sm_scale=w.sm_scale, kernel=kern).cpu()
        assert maxabs(o[:, :, rows], exact) <= TOL_F16, kern
    assert fst.last_status() == 0


def test_output_delivered_to_several_copies_of_the_full_tensor(fst):
    """fst_attention_fwd_scatter on one GPU: the "ranks'" copies of the full output are three
    tensors of this device, and a shard's rows must land in all of them at the shard's (tree, head)
    origin - by trees and by heads - leaving every other element untouched."""
    import ctypes
    from fstattention_b200 import configs

    class Copies:                                        # what sharding.GatheredOutput hands to fst_attention
        def __init__(self, tensors, rank, z0, h0):
            self.local, self.n_ranks, self.rank, self.z0, self.h0 = tensors[rank], len(tensors), rank, z0, h0
            self.pointer_array = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

    trees = configs.jittered_forest(7, 6, 256)
    T, H, N, D = len(trees), 8, 256, 128
    q, k, v = (x.cuda() for x in make_qkv(T, H, N, N, D, torch.float16, seed=71))
    meta_all = fst.build_tree_metadata(trees, 64, 64)
    for kern in ("auto", "tma_t32", "tma_t64"):
        want = fst.fst_attention(q, k, v, meta_all, sm_scale=D ** -0.5, kernel=kern)    # same tile width, same bits
        copies = [torch.full((T, H, N, D), 7.0, dtype=torch.float16, device="cuda") for _ in range(3)]
        # trees 2..3 as one shard, written by "rank" 1
        meta = fst.build_tree_metadata(trees[2:4], 64, 64)
        got = fst.fst_attention(q[2:4], k[2:4], v[2:4], meta, sm_scale=D ** -0.5, kernel=kern,
                                scatter=Copies(copies, 1, 2, 0))
        assert got.data_ptr() == copies[1].data_ptr()
        # heads 5..7 of every tree as another shard, written by "rank" 2
        fst.fst_attention(q[:, 5:8], k[:, 5:8], v[:, 5:8], meta_all, sm_scale=D ** -0.5, kernel=kern,
                          scatter=Copies(copies, 2, 0, 5))
        torch.cuda.synchronize()
        for c in copies:
            assert torch.equal(c[2:4, :5], want[2:4, :5]) and torch.equal(c[:, 5:8], want[:, 5:8]), kern
            rest = c.clone()
            rest[2:4] = 7.0
            rest[:, 5:8] = 7.0
            assert (rest == 7.0).all(), kern
    with pytest.raises(ValueError, match="shared prefix"):      # no shared prefix on this path
        fst.fst_attention(q[:1], torch.cat((k[:1], k[:1]), 2), torch.cat((v[:1], v[:1]), 2),
                          fst.build_tree_metadata(trees[0], 64, 64), sm_scale=1.0,
                          scatter=Copies(copies, 0, 0, 0))
    assert fst.last_status() == 0
