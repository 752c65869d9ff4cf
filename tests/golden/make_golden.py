"""Generate the golden fixtures in this directory from the reference implementation itself.

Run once on a machine that has the reference checkout (its path is the first argument, or the
environment variable FST_REFERENCE_DIR); the .npz files it writes are committed and are the
only thing the tests read.

  python tests/golden/make_golden.py /path/to/reference

What is recorded:
  * metadata_*.npz  - for each tree: the parent array and the outputs of the reference's own
    ``utils.create_fst_attention_kernel_inputs`` (mask bit-packed) and, for the small trees,
    ``utils.create_full_attention_mask``.
  * attention_*.npz - q/k/v plus two outputs: the reference's Triton kernel (the part of
    fstattention.py above its test code, executed by the Triton CPU interpreter) and the dense
    formula of its test (fstattention.py:216-219) evaluated on the same CPU tensors.
"""
from __future__ import annotations

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from fstattention_b200 import configs  # noqa: E402
from oracle.tree_oracle import lineage_from_parent  # noqa: E402


def load_reference(ref_dir):
    sys.path.insert(0, ref_dir)
    import utils as ref_utils  # the reference's utils.py
    src = open(os.path.join(ref_dir, "fstattention.py")).read()
    head = src.split("def test_op", 1)[0]       # kernel + wrapper only; the rest needs CUDA
    ns = {"__name__": "ref_fst_head"}
    exec(compile(head, os.path.join(ref_dir, "fstattention.py"), "exec"), ns)
    return ref_utils, ns["fst_attention"]


def metadata_case(ref_utils, parent, block_m, max_ancestors, with_full_mask):
    lin, lvl = lineage_from_parent(parent)
    out = {"parent": np.asarray(parent, np.int32), "block_m": block_m,
           "max_ancestors": max_ancestors}
    if with_full_mask:
        fm = ref_utils.create_full_attention_mask(lin.clone())
        out["full_mask_bits"] = np.packbits(fm.numpy().astype(bool), axis=1)
        out["full_mask_shape"] = np.asarray(fm.shape)
    ai, am, li = ref_utils.create_fst_attention_kernel_inputs(lin.clone(), lvl, block_m=block_m,
                                                              max_ancestors=max_ancestors)
    out["ancestor_idx"] = ai.numpy().astype(np.int32)
    out["ancestor_mask_bits"] = np.packbits(am.numpy(), axis=2)
    out["leaf_idx"] = li.numpy().astype(np.int32)
    return out


def save(name, cases):
    flat = {}
    for cname, d in cases.items():
        for key, val in d.items():
            flat[f"{cname}/{key}"] = val
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **flat)
    print("wrote", path, os.path.getsize(path), "bytes")


def dense_formula(q, k, v, mask, sm_scale):
    # the reference's in-test formula, fstattention.py:216-219, on CPU tensors
    p = torch.matmul(q, k.transpose(2, 3)) * sm_scale
    p[:, :, mask == 0] = float("-inf")
    p = torch.softmax(p.float(), dim=-1).to(q.dtype)
    return torch.matmul(p, v)


def attention_case(ref_utils, ref_attn, parent, heads, head_dim, dtype, block_m, max_ancestors,
                   seed, prefix=0, std=1.0, sm_scale=None, lineage=None):
    if lineage is None:
        lin, lvl = lineage_from_parent(parent)
    else:
        lin, lvl = lineage
    n = lin.shape[0]
    nb = -(-n // block_m)
    npad = nb * block_m
    core = ref_utils.create_full_attention_mask(lin.clone())[:n, :n]
    mask = torch.zeros((npad, npad))
    mask[:n, :n] = core
    ai, am, li = ref_utils.create_fst_attention_kernel_inputs(lin.clone(), lvl, block_m=block_m,
                                                              max_ancestors=max_ancestors)
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((1, heads, npad, head_dim), generator=g) * std).to(dtype)
    k = (torch.randn((1, heads, prefix + npad, head_dim), generator=g) * std).to(dtype)
    v = (torch.randn((1, heads, prefix + npad, head_dim), generator=g) * std).to(dtype)
    sm_scale = sm_scale if sm_scale is not None else head_dim ** -0.5
    if prefix:
        mask = torch.cat((torch.ones((npad, prefix)), mask), dim=1)
        ai = torch.where(ai >= 0, ai + prefix, ai)     # shift real entries only
        li = torch.where(li >= 0, li + prefix, li)
    dense = dense_formula(q, k, v, mask, sm_scale)
    tri = ref_attn(q, k, v, ai, am, li, sm_scale, BLOCK_M=block_m, MAX_ANCESTORS=max_ancestors)
    return {"parent": np.asarray(parent, np.int32), "n": n, "block_m": block_m,
            "max_ancestors": max_ancestors, "prefix": prefix, "sm_scale": np.float64(sm_scale),
            "q": q.numpy(), "k": k.numpy(), "v": v.numpy(),
            "out_dense": dense.float().numpy().astype(q.numpy().dtype),
            "out_triton": tri.float().numpy().astype(q.numpy().dtype)}


def parent_of_reference_tree(ref_utils, depth):
    lin, lvl = ref_utils.create_tree(depth=depth)
    n = lin.shape[0]
    par = np.full(n, -1, np.int64)
    nz = lvl.numpy() > 0
    par[nz] = lin.numpy()[np.arange(n)[nz], lvl.numpy()[nz] - 1]
    return par.tolist(), (lin, lvl)


def main():
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FST_REFERENCE_DIR")
    if not ref_dir:
        raise SystemExit("usage: make_golden.py <reference checkout>")
    ref_utils, ref_attn = load_reference(ref_dir)

    meta = {}
    meta["binary31_bm16"] = metadata_case(ref_utils, configs.binary_tree(31), 16, 16, True)
    meta["medusa256_bm64"] = metadata_case(ref_utils, configs.left_weighted_tree(), 64, 64, True)
    meta["medusa256_bm128"] = metadata_case(ref_utils, configs.left_weighted_tree(), 128, 64, False)
    for s in range(3):
        meta[f"random1024_s{s}_bm64"] = metadata_case(
            ref_utils, configs.random_window_tree(s), 64, 256, False)
    forest = configs.jittered_forest(0, 64, 256)
    for t in (0, 1, 31, 63):
        meta[f"forest64_t{t}_bm64"] = metadata_case(ref_utils, forest[t], 64, 64, False)
    meta["deep4096_bm64"] = metadata_case(ref_utils, configs.deep_chain_tree(0, 4096), 64, 128, False)
    meta["deep4096_bm128"] = metadata_case(ref_utils, configs.deep_chain_tree(0, 4096), 128, 192, False)
    meta["deep2579_literal_bm64"] = metadata_case(
        ref_utils, configs.deep_chain_tree(0, 4096, chains=64), 64, 128, False)
    par7, _ = parent_of_reference_tree(ref_utils, 7)          # the reference's own fixture tree
    meta["reftree_d7_bm128"] = metadata_case(ref_utils, par7, 128, 64, False)
    meta["reftree_d7_bm64"] = metadata_case(ref_utils, par7, 64, 32, False)
    par3, _ = parent_of_reference_tree(ref_utils, 3)
    meta["reftree_d3_bm32"] = metadata_case(ref_utils, par3, 32, 32, True)
    # multi-root forest with an irregular tail and a partial last block
    rng = np.random.RandomState(7)
    par = [-1, -1, -1] + [int(rng.randint(-1, i)) for i in range(3, 157)]
    meta["multiroot157_bm32"] = metadata_case(ref_utils, par, 32, 64, True)
    meta["single_node_bm16"] = metadata_case(ref_utils, [-1], 16, 16, True)
    meta["chain40_bm16"] = metadata_case(ref_utils, [-1] + list(range(39)), 16, 64, True)
    save("metadata_golden.npz", meta)

    att = {}
    att["binary31_fp32"] = attention_case(ref_utils, ref_attn, configs.binary_tree(31), 4, 64,
                                          torch.float32, 16, 16, seed=0)
    att["medusa256_fp16_h2"] = attention_case(ref_utils, ref_attn, configs.left_weighted_tree(),
                                              2, 128, torch.float16, 64, 64, seed=1)
    att["medusa256_fp16_d64_bm128"] = attention_case(
        ref_utils, ref_attn, configs.left_weighted_tree(), 2, 64, torch.float16, 128, 64, seed=2)
    par5, lin5 = parent_of_reference_tree(ref_utils, 5)        # 252 nodes -> padded to 256
    att["reftree_d5_prefix128"] = attention_case(
        ref_utils, ref_attn, par5, 2, 64, torch.float16, 128, 64, seed=20, prefix=128,
        std=0.5, sm_scale=0.5, lineage=lin5)
    att["reftree_d5_noprefix"] = attention_case(
        ref_utils, ref_attn, par5, 2, 64, torch.float16, 128, 64, seed=20, prefix=0,
        std=0.5, sm_scale=0.5, lineage=lin5)
    save("attention_golden.npz", att)


if __name__ == "__main__":
    main()
