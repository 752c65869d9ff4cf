"""The allocation-free entry point, called through the C ABI, against the workspace one.

fst_attention_fwd_ref_static exists for hosts that may not allocate device memory where the
attention runs (an engine's plugin hook, a serving loop that owns all device memory through its
own pool): it keeps its scratch in a fixed array inside the library.  It must give exactly what
fst_attention_fwd_ref gives with a caller-provided workspace, call after call, because every
call shares that one array.  This file sorts last on purpose so that a run that stops at the
first failure has already run everything else.
"""
import pytest
import torch

from conftest import unpack_golden_metadata

pytestmark = pytest.mark.gpu

TOL_F16 = 2e-3      # the attention tests' fp16 gate; the two entry points are expected to agree exactly


def _call(lib, fn_name, q, k, v, ai, am, li, bm, ma, scale, workspace=None):
    o = torch.full_like(q, float("nan"))
    status = torch.zeros(4, dtype=torch.int32, device=q.device)
    Z, H, n_q, D = q.shape
    args = [q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), None,
            ai.data_ptr(), am.data_ptr(), li.data_ptr(), 1, Z, H, n_q, k.shape[2], D,
            *q.stride()[:3], *k.stride()[:3], *v.stride()[:3], *o.stride()[:3],
            bm, ma, scale, 0, 0]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    args += [status.data_ptr(), torch.cuda.current_stream().cuda_stream]
    fn = getattr(lib, fn_name)
    torch.cuda.synchronize()
    before = (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0])
    rc = fn(*args)
    torch.cuda.synchronize()
    after = (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0])
    _call.device_memory_moved = after != before          # by the library call alone: no tensor is made or dropped in between
    return rc, o, status


def test_static_scratch_entry_matches_workspace_entry(built_lib, metadata_golden):
    from fstattention_b200 import _lib
    lib = _lib.lib()
    cases = [("medusa256_bm64", 4, 128, 0), ("random1024_s2_bm64", 2, 128, 64)]
    for round_no in range(2):                        # two calls in a row reuse the same array
        for name, heads, d, prefix in cases:
            ai, am, li, bm, ma = unpack_golden_metadata(metadata_golden[name])
            n = len(metadata_golden[name]["parent"])
            g = torch.Generator().manual_seed(100 + round_no)
            q = torch.randn((1, heads, n, d), generator=g).half().cuda()
            k = torch.randn((1, heads, prefix + n, d), generator=g).half().cuda()
            v = torch.randn((1, heads, prefix + n, d), generator=g).half().cuda()
            d_ai, d_am, d_li = (ai + prefix).cuda(), am.cuda(), (li + prefix).cuda()
            need = lib.fst_attention_ref_workspace_bytes(1, n, bm, ma)
            assert need <= _lib.STATIC_SCRATCH_BYTES
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            rc_a, want, st_a = _call(lib, "fst_attention_fwd_ref", q, k, v, d_ai, d_am, d_li, bm, ma,
                                     d ** -0.5, workspace=ws)
            rc_b, got, st_b = _call(lib, "fst_attention_fwd_ref_static", q, k, v, d_ai, d_am, d_li, bm, ma,
                                    d ** -0.5)
            torch.cuda.synchronize()
            if round_no == 1:                            # warmed up: the call took and gave back no device memory
                assert not _call.device_memory_moved
            assert rc_a == 0 and rc_b == 0
            assert st_a[0].item() == 0 and st_b[0].item() == 0
            assert torch.isfinite(got).all()
            assert (got.float() - want.float()).abs().max().item() <= TOL_F16, (name, round_no)
            assert torch.equal(got, want), (name, round_no)


def test_static_scratch_entry_refuses_oversized_metadata(built_lib):
    from fstattention_b200 import _lib
    lib = _lib.lib()
    bm, ma, n = 64, 4096, 8192                       # packed form needs several MB
    assert lib.fst_attention_ref_workspace_bytes(1, n, bm, ma) > _lib.STATIC_SCRATCH_BYTES
    q = torch.zeros((1, 1, n, 64), dtype=torch.float16, device="cuda")
    nb = n // bm
    ai = torch.full((nb, ma), -1, dtype=torch.long, device="cuda")
    am = torch.zeros((nb, bm, ma), dtype=torch.bool, device="cuda")
    li = torch.full((nb, bm), -1, dtype=torch.long, device="cuda")
    rc, o, status = _call(lib, "fst_attention_fwd_ref_static", q, q, q, ai, am, li, bm, ma, 1.0)
    torch.cuda.synchronize()
    assert rc == 6 and "scratch" in _lib.status_string(rc)
    assert torch.isnan(o).all()                      # nothing was launched
