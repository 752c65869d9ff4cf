"""The CPU oracle against fixtures produced by the reference itself (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from conftest import unpack_golden_metadata
from oracle import tree_oracle as orc


def test_metadata_matches_reference_bit_exact(metadata_golden):
    assert len(metadata_golden) >= 15
    for name, case in metadata_golden.items():
        ai, am, li, bm, ma = unpack_golden_metadata(case)
        lin, lvl = orc.lineage_from_parent(case["parent"].tolist())
        lin0 = lin.clone()
        o_ai, o_am, o_li = orc.block_metadata(lin, lvl, bm, ma)
        assert torch.equal(lin, lin0), name          # oracle leaves its input alone
        assert o_ai.dtype == torch.long and o_am.dtype == torch.bool and o_li.dtype == torch.long
        assert torch.equal(o_ai, ai), name
        assert torch.equal(o_am, am), name
        assert torch.equal(o_li, li), name


def test_full_mask_matches_reference(metadata_golden):
    seen = 0
    for name, case in metadata_golden.items():
        if "full_mask_bits" not in case:
            continue
        shape = tuple(case["full_mask_shape"])
        ref = np.unpackbits(case["full_mask_bits"], axis=1)[:, : shape[1]].astype(np.float32)
        lin, _ = orc.lineage_from_parent(case["parent"].tolist())
        got = orc.full_attention_mask(lin)           # default pad of 4, float32, as the reference
        assert got.dtype == torch.float32 and tuple(got.shape) == shape, name
        assert np.array_equal(got.numpy(), ref), name
        seen += 1
    assert seen >= 5


def test_metadata_overflow_raises_like_reference(metadata_golden):
    case = metadata_golden["medusa256_bm64"]
    lin, lvl = orc.lineage_from_parent(case["parent"].tolist())
    with pytest.raises(RuntimeError):
        orc.block_metadata(lin, lvl, 64, 16)


def test_parent_lineage_round_trip(metadata_golden):
    for name, case in metadata_golden.items():
        par = case["parent"].astype(np.int64)
        lin, lvl = orc.lineage_from_parent(par.tolist())
        assert np.array_equal(orc.parent_from_lineage(lin, lvl).numpy(), par), name


def test_mask_equals_metadata_attention_sets(metadata_golden):
    """The block metadata and the dense mask describe the same attention sets."""
    for name in ("binary31_bm16", "multiroot157_bm32", "chain40_bm16"):
        case = metadata_golden[name]
        ai, am, li, bm, ma = unpack_golden_metadata(case)
        lin, _ = orc.lineage_from_parent(case["parent"].tolist())
        n = lin.shape[0]
        dense = orc.full_attention_mask(lin, pad_rows=0).numpy().astype(bool)
        for k in range(n):
            b, j = divmod(k, bm)
            cols = set(ai[b][am[b, j]].tolist())
            if li[b, j] >= 0:
                cols.add(int(li[b, j]))
            assert cols == set(np.nonzero(dense[k])[0].tolist()), (name, k)


def _tol(dtype):
    # fp16 cases: the reference's own test tolerance (atol 1e-2, rtol 0); fp32: rounding only
    return 1e-2 if dtype == np.float16 else 2e-5


def test_dense_attention_matches_reference_outputs(attention_golden):
    for name, case in attention_golden.items():
        q, k, v = (torch.from_numpy(case[x]) for x in ("q", "k", "v"))
        n, bm, prefix = int(case["n"]), int(case["block_m"]), int(case["prefix"])
        out = orc.tree_attention_reference(q, k, v, case["parent"].tolist(), float(case["sm_scale"]),
                                           bm, prefix_len=prefix)
        got = out[:, :, :n].float().numpy()
        dense = case["out_dense"][:, :, :n].astype(np.float32)
        tri = case["out_triton"][:, :, :n].astype(np.float32)
        # same formula, same library: identical to the reference's dense evaluation
        assert np.array_equal(got, dense), name
        # and within the reference test's tolerance of the reference kernel
        assert np.abs(got - tri).max() <= _tol(case["q"].dtype), name


def test_upcast_oracle_is_closer_to_reference_kernel(attention_golden):
    case = attention_golden["medusa256_fp16_h2"]
    q, k, v = (torch.from_numpy(case[x]) for x in ("q", "k", "v"))
    n = int(case["n"])
    o32 = orc.tree_attention_reference(q, k, v, case["parent"].tolist(), float(case["sm_scale"]),
                                       int(case["block_m"]), compute_dtype=torch.float32)
    tri = case["out_triton"][:, :, :n].astype(np.float32)
    assert np.abs(o32[:, :, :n].numpy() - tri).max() < 4e-3
