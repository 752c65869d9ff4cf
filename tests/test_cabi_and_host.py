"""CPU-only checks: the library loads and exports the header's symbols; host-side logic."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "fstattn_b200.h")).read()
    code = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(fst_[a-z_0-9]+)\s*\(", code))
    assert len(declared) >= 8
    lib = ctypes.CDLL(built_lib)
    for name in declared:
        assert hasattr(lib, name), name
    from fstattention_b200 import _lib
    assert set(_lib.EXPORTS) == declared


def test_bindings_match_the_header(built_lib):
    """Every ctypes prototype has as many arguments, of the right kind, as the header declares."""
    import ctypes as C
    header = open(os.path.join(ROOT, "include", "fstattn_b200.h")).read()
    code = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    from fstattention_b200 import _lib
    lib = _lib.lib()
    kinds = {"int": C.c_int, "int64_t": C.c_int64, "size_t": C.c_size_t, "float": C.c_float,
             "double": C.c_double}
    for name, params in re.findall(r"\b(fst_[a-z_0-9]+)\s*\(([^)]*)\)\s*;", code):
        params = params.strip()
        want = []
        if params != "void":
            for prm in params.split(","):
                prm = " ".join(prm.split())
                if "*" in prm:
                    want.append(C.c_void_p)
                else:
                    want.append(kinds[prm.rsplit(" ", 1)[0].replace("const ", "")])
        got = list(getattr(lib, name).argtypes)
        got = [C.c_void_p if t in (C.c_char_p,) else t for t in got]
        assert got == want, (name, len(got), len(want))


def test_host_only_entry_points(built_lib):
    from fstattention_b200 import _lib
    lib = _lib.lib()
    assert lib.fst_version() == 100
    assert "max_ancestors" in _lib.status_string(17)
    assert _lib.status_string(0) == "ok"
    # layout: count | idx | emask | bmask, every part 16-byte aligned
    assert lib.fst_packed_meta_bytes(4, 64, 64) == 16 + 4 * 64 * 4 + 4 * 64 * 2 * 4 + 4 * 64 * 2 * 4
    assert lib.fst_packed_meta_bytes(0, 64, 64) == 0
    assert lib.fst_attention_ref_workspace_bytes(2, 256, 64, 64) == 2 * lib.fst_packed_meta_bytes(4, 64, 64)
    # the device-built forest has the reference's node counts (utils.py:27-40: 2^(depth+3) - 4)
    for depth in (5, 7, 9):
        assert lib.fst_tree_topk_nodes(depth, 4, 0.5) == 2 ** (depth + 3) - 4
    assert lib.fst_tree_topk_nodes(14, 4, 0.5) == -1          # a level of 32768 nodes: beyond the kernel
    assert lib.fst_tree_topk_nodes(7, 4, 1.5) == -1
    assert lib.fst_build_tree_topk(None, 1, 7, 4, 0.5, 1020, None, None, None, None) == 1
    assert lib.fst_build_tree_topk(ctypes.c_void_p(256), 1, 14, 4, 0.5, 1 << 20, ctypes.c_void_p(256), None, None, None) == 6
    assert lib.fst_attention_fwd_scatter(None, None, None, None, 2, 0, 0, 0, 2, 2, None, None, 0, 1, 1, 4, 4, 64,
                                         *([1] * 12), 64, 64, 1.0, 0, 0, None, None) == 1
    # argument checks happen before any CUDA call
    assert lib.fst_precompute(None, 1, 4, 16, 16, None, None, None, None, 0, None, None) == 1
    assert lib.fst_precompute(ctypes.c_void_p(256), 1, 1 << 20, 16, 16, None, None, None, None, 0, None, None) == 6


def test_packed_layout_helper_agrees_with_library(built_lib):
    from fstattention_b200 import _lib
    from helpers import packed_offsets
    lib = _lib.lib()
    for nb, bm, ma in [(1, 16, 16), (4, 64, 64), (16, 64, 256), (64, 64, 128), (33, 128, 192), (3, 24, 40)]:
        assert packed_offsets(nb, bm, ma)[3] == lib.fst_packed_meta_bytes(nb, bm, ma)


def test_cpu_tensors_are_refused():
    import fstattention_b200 as fst
    q = torch.zeros(1, 1, 16, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fst.fst_attention(q, q, q, q.long(), q.bool(), q.long(), 1.0)
    with pytest.raises(AssertionError):
        fst.fst_attention(q[..., :48], q[..., :48], q[..., :48], None, None, None, 1.0)


def test_lineage_adapters_round_trip(metadata_golden):
    import fstattention_b200 as fst
    from oracle import tree_oracle as orc
    for name in ("binary31_bm16", "multiroot157_bm32", "reftree_d3_bm32", "medusa256_bm64"):
        par = metadata_golden[name]["parent"].tolist()
        lin, lvl = fst.lineage_from_parent(par)
        o_lin, o_lvl = orc.lineage_from_parent(par)
        assert torch.equal(lin, o_lin) and torch.equal(lvl, o_lvl)
        assert fst.parent_from_lineage(lin, lvl).tolist() == par
    with pytest.raises(ValueError):
        fst.lineage_from_parent([-1, 2, 0])


def test_workload_definitions():
    from fstattention_b200 import configs
    w = configs.workload("medusa256")
    assert len(w.trees[0]) == 256 and w.heads == 32 and w.head_dim == 128 and w.block_m == 64
    depth = [0] * 256
    for i, p in enumerate(w.trees[0]):
        depth[i] = 0 if p < 0 else depth[p] + 1
    assert np.bincount(depth).tolist() == [1, 10, 36, 133, 76]
    assert configs.workload("binary31").trees[0][:5] == [-1, 0, 0, 1, 1]
    assert configs.workload("random1024", 3).trees[0] == configs.random_window_tree(3)
    assert configs.workload("random1024", 3).trees[0] != configs.random_window_tree(4)
    forest = configs.workload("forest64").trees
    assert len(forest) == 64 and all(len(t) == 256 for t in forest)
    deep = configs.workload("deep4096").trees[0]
    assert len(deep) == 4096 and all(p < i for i, p in enumerate(deep))
    assert len(configs.deep_chain_tree(0, 4096, chains=64)) == 2579


def test_create_tree_and_full_mask_match_reference(metadata_golden):
    """Fixture generator and dense mask builder against what the reference produced."""
    import fstattention_b200 as fst
    from oracle import tree_oracle as orc
    for depth, key in ((3, "reftree_d3_bm32"), (7, "reftree_d7_bm128")):
        case = metadata_golden[key]
        lin, lvl = fst.create_tree(depth=depth)
        ref_lin, ref_lvl = orc.lineage_from_parent(case["parent"].tolist())
        assert lin.dtype == torch.long and lvl.dtype == torch.long
        assert lin.shape == (2 ** (depth + 3) - 4, depth + 1)
        assert torch.equal(lin, ref_lin) and torch.equal(lvl, ref_lvl)
    assert fst.DEPTH_MAPPING[2 ** 11] == 8 and fst.MAX_ANCESTOR_MAPPING[2 ** 16] == 64
    seen = 0
    for name, case in metadata_golden.items():
        if "full_mask_bits" not in case:
            continue
        shape = tuple(case["full_mask_shape"])
        ref = np.unpackbits(case["full_mask_bits"], axis=1)[:, : shape[1]].astype(np.float32)
        lin, _ = orc.lineage_from_parent(case["parent"].tolist())
        got = fst.create_full_attention_mask(lin)
        assert got.dtype == torch.float32 and tuple(got.shape) == shape
        assert np.array_equal(got.numpy(), ref), name
        seen += 1
    assert seen >= 5


def _gathered_rows(parent, bm):
    total = 0
    for lo in range(0, len(parent), bm):
        anc = set()
        rows = range(lo, min(lo + bm, len(parent)))
        for k in rows:
            x = parent[k]
            while x >= 0 and x not in anc:
                anc.add(x)
                x = parent[x]
        total += len(anc) + sum(1 for k in rows if k not in anc)
    return total


def test_dfs_order_is_a_valid_renumbering_and_shrinks_the_gather():
    import fstattention_b200 as fst
    from fstattention_b200 import configs
    deep = configs.deep_chain_tree(0, 4096, chains=64)          # 2579 nodes, construction order
    # breadth-first numbering of the same tree: the bad case
    children = [[] for _ in deep]
    for i, p in enumerate(deep):
        if p >= 0:
            children[p].append(i)
    bfs = [0]
    for x in bfs:
        bfs.extend(children[x])
    new_of = {old: new for new, old in enumerate(bfs)}
    bfs_parent = [-1 if deep[old] < 0 else new_of[deep[old]] for old in bfs]
    for par in (bfs_parent, deep, configs.random_window_tree(1, 500), [-1, -1, 0, 1, 0, -1, 5]):
        order, new_parent = fst.dfs_order(par)
        n = len(par)
        assert sorted(order) == list(range(n))
        assert all(p < i for i, p in enumerate(new_parent))
        pos = {old: new for new, old in enumerate(order)}
        for new, old in enumerate(order):                        # same tree, renamed
            assert new_parent[new] == (-1 if par[old] < 0 else pos[par[old]])
        # pre-order: every subtree is a contiguous run starting at its root
        last = list(range(n))
        for i in range(n - 1, -1, -1):
            if new_parent[i] >= 0:
                last[new_parent[i]] = max(last[new_parent[i]], last[i])
        size = [1] * n
        for i in range(n - 1, -1, -1):
            if new_parent[i] >= 0:
                size[new_parent[i]] += size[i]
        assert all(last[i] == i + size[i] - 1 for i in range(n))
    order, dfs_parent = fst.dfs_order(bfs_parent)
    assert _gathered_rows(dfs_parent, 64) * 5 < _gathered_rows(bfs_parent, 64)


@pytest.mark.gpu
def test_c_program_against_the_library(built_lib, tmp_path):
    """tests/cabi/cabi_example.cu - a caller with no Python and no torch - builds against the header
    and the shared library, runs precompute + attention and agrees with its own host loop."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path / "cabi_example")
    libdir = os.path.dirname(built_lib)
    subprocess.run([nvcc, "-O2", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cabi", "cabi_example.cu"),
                    "-L", libdir, "-lfstattn_b200", "-Xlinker", "-rpath", "-Xlinker", libdir, "-o", exe],
                   check=True, capture_output=True, timeout=300)
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "max-abs difference" in run.stdout
    assert "host time per fst_attention_fwd call" in run.stdout
    print(run.stdout)
