"""Attention entry point: the reference's ``fst_attention`` on the sm_100a kernels.

Same positional signature as fstattention.py:153 of the reference::

    o = fst_attention(q, k, v, ancestor_idx, ancestor_mask, leaf_idx, sm_scale,
                      BLOCK_M=128, MAX_ANCESTORS=64)

``q`` is ``[Z, H, N, D]``, ``k``/``v`` are ``[Z, H, P + N, D]`` where the first ``P`` rows are a
prefix every query attends to.  The launch is asynchronous on torch's current stream.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib
from .utils import TreeMetadata, metadata_of

_DTYPES = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16,
           torch.float32: _lib.DTYPE_F32}
_status = {}


def _status_record(device) -> torch.Tensor:
    rec = _status.get(device)
    if rec is None:
        rec = _status[device] = torch.zeros(_lib.STATUS_WORDS, dtype=torch.int32, device=device)
    return rec


def _resolve(device) -> torch.device:
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def last_status(device=None, clear: bool = False) -> int:
    """Device-side status code recorded by attention launches on ``device`` (synchronises).

    The record keeps the first problem it saw until it is cleared: pass ``clear=True`` (or call
    ``clear_status``) once the code has been dealt with, so that later launches report afresh."""
    rec = _status.get(_resolve(device))
    if rec is None:
        return 0
    code = int(rec[0].item())
    if clear and code != 0:
        rec.zero_()
    return code


def clear_status(device=None) -> None:
    """Zero the status record of ``device`` (asynchronous, on the current stream)."""
    rec = _status.get(_resolve(device))
    if rec is not None:
        rec.zero_()


def _strides(t):
    st = t.stride()
    if st[3] != 1:
        raise ValueError("the head dimension must be contiguous")
    return [st[0], st[1], st[2]]


def _raw_stream(dev) -> int:
    """Handle of torch's current stream on ``dev`` (the private fast path when torch has it:
    this sits on the per-layer call path of an eager decoder)."""
    try:
        return torch._C._cuda_getCurrentRawStream(dev.index)
    except AttributeError:
        return torch.cuda.current_stream(dev).cuda_stream


class _OnDevice:
    """``torch.cuda.device(dev)`` that does nothing when ``dev`` is already current."""

    def __init__(self, dev):
        self.ctx = None if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


_SMS = {}


def _pick_splits(kv_splits, q, prefix, block_m, kernel):
    """(runs the shared prefix is cut into, whether a workspace is needed).

    Only the tensor-core kernels split.  With head_dim 64 or 128 and at least 256 prefix rows the
    prefix goes to the tcgen05 kernel: one CTA per 128 query rows, head, batch element and run.
    Its shared memory allows one CTA per SM, so the automatic choice is as many runs as keep the
    grid within one wave, each at least 256 rows.  Otherwise the tree kernel walks the prefix
    itself, split to about four CTAs per SM."""
    if q.dtype not in (torch.float16, torch.bfloat16) or q.shape[-1] not in (64, 128) \
            or block_m not in (32, 64, 128) or kernel in ("simt", "mma") or prefix <= 0:
        return 1, False
    dev = q.device
    sms = _SMS.get(dev)
    if sms is None:
        sms = _SMS[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    z_cap = 65535 // max(q.shape[0], 1)
    if q.shape[-1] in (64, 128) and (kernel == "tma_umma" or (kernel == "auto" and prefix >= 256)):
        if kv_splits is not None:
            return max(1, min(int(kv_splits), z_cap)), True
        ctas = q.shape[0] * q.shape[1] * -(-q.shape[2] // 128)
        return int(max(1, min(sms // max(ctas, 1), prefix // 256, z_cap))), True
    if kv_splits is not None:
        splits = max(1, min(int(kv_splits), z_cap))
        return splits, splits > 1
    ctas = q.shape[0] * q.shape[1] * -(-q.shape[2] // block_m)
    splits = int(max(1, min((4 * sms) // max(ctas, 1), prefix // 512, z_cap)))
    return splits, splits > 1


def launch_plan(q, prefix, block_m, kernel: str = "auto", kv_splits: Optional[int] = None) -> dict:
    """Which kernels one ``fst_attention`` call on packed metadata launches for ``q`` (shape and
    dtype only), a shared prefix of ``prefix`` rows and the given block size, mirroring the
    dispatch inside the library: ``{"kernels": [...], "prefix_runs": r}``."""
    splits, need_ws = _pick_splits(kv_splits, q, prefix, block_m, kernel)
    tensor_core = q.dtype in (torch.float16, torch.bfloat16) and q.shape[-1] in (64, 128) \
        and block_m in (16, 32, 64, 128)
    tree = "attn_simt_kernel" if kernel == "simt" or not tensor_core else \
        "attn_mma_kernel" if kernel == "mma" or block_m == 16 else "attn_tma_kernel"
    if kernel == "persist" and tree == "attn_tma_kernel" and prefix == 0 and block_m in (64, 128):
        tree = "attn_persist_kernel"                      # by hand only: it measured slower than attn_tma_kernel
    if need_ws and q.shape[-1] in (64, 128) and (kernel == "tma_umma" or (kernel == "auto" and prefix >= 256)):
        return {"kernels": ["prefix_umma_kernel", tree, "combine_splits_kernel"], "prefix_runs": splits}
    if need_ws:
        return {"kernels": [tree, "combine_splits_kernel"], "prefix_runs": splits}
    return {"kernels": [tree], "prefix_runs": 1}


def fst_attention(q, k, v, ancestor_idx, ancestor_mask=None, leaf_idx=None, sm_scale=None,
                  BLOCK_M=128, MAX_ANCESTORS=64, *, out: Optional[torch.Tensor] = None,
                  return_lse: bool = False, kernel: str = "auto", kv_splits: Optional[int] = None,
                  scatter=None):
    """Fused sparse tree attention forward.

    ``ancestor_idx, ancestor_mask, leaf_idx`` are the tensors returned by
    ``create_fst_attention_kernel_inputs`` (from this package, or the reference's moved to the
    GPU) built with ``block_m=BLOCK_M`` and ``max_ancestors=MAX_ANCESTORS``; index tensors hold
    absolute K/V rows, i.e. the caller adds the prefix length as fstattention.py:211-212 does.
    Alternatively pass a ``TreeMetadata`` as ``ancestor_idx`` and leave the other two ``None``;
    its block size and ancestor bound are used.  Metadata with a leading tree dimension of size
    ``Z`` gives every batch element its own tree.  ``k`` and ``v`` may have fewer heads than ``q``
    (grouped-query attention, ``H`` a multiple of ``H_kv``).

    ``kv_splits`` cuts a shared prefix into that many runs handled by separate CTAs and merged
    afterwards; ``None`` picks a split that fills the GPU when the tree alone does not.

    ``scatter`` (see ``sharding.GatheredOutput.target``) makes the kernel deliver this call's
    rows into every rank's copy of a full output tensor instead of a local ``out``; the return
    value is then this rank's copy, complete only after the ranks have met.

    Asserts like the reference (fstattention.py:155-157): equal head dims, in {16, 32, 64, 128}.
    """
    if sm_scale is None:
        raise TypeError("sm_scale is required")
    Lq, Lk, Lv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Lq == Lk and Lk == Lv
    assert Lk in {16, 32, 64, 128}
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("fst_attention runs on CUDA tensors only; there is no CPU path")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one dtype out of float16, bfloat16, float32")
    Z, H, n_q, D = q.shape
    n_kv, H_kv = k.shape[2], k.shape[1]
    if k.shape != (Z, H_kv, n_kv, D) or v.shape != k.shape or n_kv < n_q or H_kv < 1 or H % H_kv:
        raise ValueError("k and v must be [Z, H_kv, P + N, D] with P >= 0 and H a multiple of H_kv")
    if scatter is not None:
        if out is not None:
            raise ValueError("out= and scatter= exclude each other")
        o = scatter.local
        if o.dtype != q.dtype or o.shape[2:] != q.shape[2:] or not o.is_cuda:
            raise ValueError("the gathered output must have q's dtype, rows and head dimension")
    else:
        o = torch.empty_like(q) if out is None else out
        if o.shape != q.shape or o.dtype != q.dtype or not o.is_cuda:
            raise ValueError("out must match q")
    lse = torch.empty((Z * H, n_q), device=q.device, dtype=torch.float32) if return_lse else None

    lib = _lib.lib()
    dev = q.device
    status = _status_record(dev)
    stream = _raw_stream(dev)
    kern = _lib.KERNELS[kernel]
    if not math.isfinite(sm_scale):
        raise ValueError("sm_scale must be finite")
    common_shape = [Z, H, n_q, n_kv, D] + _strides(q) + _strides(k) + _strides(v) + _strides(o)

    meta = ancestor_idx if isinstance(ancestor_idx, TreeMetadata) else \
        metadata_of(ancestor_idx, ancestor_mask, leaf_idx)
    with _OnDevice(dev):
        if meta is not None:
            if meta.n_trees not in (1, Z):
                raise ValueError("metadata must describe one tree or one tree per batch element")
            if isinstance(ancestor_idx, TreeMetadata):
                BLOCK_M, MAX_ANCESTORS = meta.block_m, meta.max_ancestors
            elif (meta.block_m, meta.max_ancestors) != (BLOCK_M, MAX_ANCESTORS):
                raise ValueError("BLOCK_M / MAX_ANCESTORS differ from the ones the metadata was built with")
            if meta.n_blocks != -(-n_q // BLOCK_M):
                raise ValueError("metadata block count does not match q")
            packed_ptr, packed_stride = meta.packed.data_ptr(), (meta.tree_stride if meta.n_trees > 1 else 0)
            # From the second launch after the precompute on, the launch ahead of this one in
            # the stream cannot be the metadata's writer: the kernel may then fetch its index
            # lists while that launch drains (FST_KERNEL_FLAG_META_STABLE).
            if meta.reads_since_build > 0:
                kern |= _lib.KERNEL_FLAG_META_STABLE
            meta.reads_since_build += 1
        else:
            # the reference's three tensors (fstattention.py:153): packed here, one more launch,
            # with the prefix length as index base (its test shifts the indices, sentinels included)
            ai, am, li = ancestor_idx, ancestor_mask, leaf_idx
            if am is None or li is None:
                raise TypeError("ancestor_mask and leaf_idx are required with plain tensors")
            if not (ai.is_cuda and am.is_cuda and li.is_cuda):
                raise RuntimeError("metadata tensors must be on the GPU (call .to('cuda') as the reference does)")
            nb = -(-n_q // BLOCK_M)
            n_meta = ai.shape[0] if ai.dim() == 3 else 1
            if tuple(ai.shape[-2:]) != (nb, MAX_ANCESTORS) or tuple(am.shape[-3:]) != (nb, BLOCK_M, MAX_ANCESTORS) \
                    or tuple(li.shape[-2:]) != (nb, BLOCK_M):
                raise ValueError("metadata shapes do not match BLOCK_M / MAX_ANCESTORS / q")
            if ai.dtype != torch.long or li.dtype != torch.long or am.dtype not in (torch.bool, torch.uint8):
                raise TypeError("metadata dtypes must be int64 / bool / int64")
            if n_meta not in (1, Z):
                raise ValueError("metadata must describe one tree or one tree per batch element")
            ai, am, li = ai.contiguous(), am.contiguous(), li.contiguous()
            stride = int(lib.fst_packed_meta_bytes(nb, BLOCK_M, MAX_ANCESTORS))
            packed = torch.empty((n_meta, stride), dtype=torch.uint8, device=dev)
            rc = lib.fst_pack_metadata(ai.data_ptr(), am.data_ptr(), li.data_ptr(), n_meta, nb, BLOCK_M,
                                       MAX_ANCESTORS, n_kv - n_q, packed.data_ptr(), stride,
                                       status.data_ptr(), stream)
            _lib.check(rc, "fst_pack_metadata")
            packed_ptr, packed_stride = packed.data_ptr(), (stride if n_meta > 1 else 0)
        splits, need_ws = _pick_splits(kv_splits, q, n_kv - n_q, BLOCK_M, kernel)
        ws, ws_bytes = None, 0
        if need_ws:
            ws_bytes = int(lib.fst_attention_split_workspace_bytes(Z, H, n_q, D, splits))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        tail = (BLOCK_M, MAX_ANCESTORS, float(sm_scale), _DTYPES[q.dtype], kern, splits,
                ws.data_ptr() if ws is not None else None, ws_bytes, status.data_ptr(), stream)
        head = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                lse.data_ptr() if lse is not None else None, packed_ptr, packed_stride)
        if scatter is not None:
            if H_kv != H or n_kv != n_q:
                raise ValueError("scatter= takes neither grouped-query heads nor a shared prefix")
            rc = lib.fst_attention_fwd_scatter(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), scatter.pointer_array, scatter.n_ranks, scatter.rank,
                scatter.z0, scatter.h0, o.shape[0], o.shape[1], lse.data_ptr() if lse is not None else None,
                packed_ptr, packed_stride, *common_shape, BLOCK_M, MAX_ANCESTORS, float(sm_scale),
                _DTYPES[q.dtype], kern, status.data_ptr(), stream)
        elif H_kv == H:
            rc = lib.fst_attention_fwd_splitkv(*head, *common_shape, *tail)
        else:                                             # grouped-query attention
            rc = lib.fst_attention_fwd_gqa(*head, Z, H, H_kv, *common_shape[2:], *tail)
        _lib.check(rc, "fst_attention_fwd")
    return (o, lse) if return_lse else o


def fst_attention_paged(q, k_tree, v_tree, meta: TreeMetadata, k_pool, v_pool, block_table, prefix_lens,
                        sm_scale, *, max_prefix: Optional[int] = None, pool_layout: str = "NHD",
                        kv_splits: Optional[int] = None, out: Optional[torch.Tensor] = None,
                        return_lse: bool = False):
    """Tree attention behind a prefix held in a paged KV cache (head_dim 64 or 128, fp16 / bf16).

    ``q`` is ``[Z, H, N, D]``; ``k_tree``, ``v_tree`` are the tree nodes' own K/V rows,
    ``[Z, H_kv, N, D]``.  The prefix of batch element ``z`` is rows ``[0, prefix_lens[z])`` of
    the sequence whose pages ``block_table[z]`` lists (int32, on the GPU, as is ``prefix_lens``):
    row ``r`` lives in page ``block_table[z, r // page_size]``.  The pools are
    ``[n_pages, page_size, H_kv, D]`` (``pool_layout="NHD"``) or ``[n_pages, H_kv, page_size, D]``
    (``"HND"``), page_size 16, 32, 64 or 128.  ``max_prefix`` (default: the largest entry of
    ``prefix_lens``, which costs a device synchronisation) sizes the grid.  ``meta`` is the
    ``TreeMetadata`` of the tree (``build_tree_metadata``)."""
    if not isinstance(meta, TreeMetadata):
        raise TypeError("meta must be a TreeMetadata (build_tree_metadata)")
    if not all(t.is_cuda for t in (q, k_tree, v_tree, k_pool, v_pool, block_table, prefix_lens)):
        raise RuntimeError("fst_attention_paged runs on CUDA tensors only; there is no CPU path")
    if q.dtype not in (torch.float16, torch.bfloat16) or any(t.dtype != q.dtype for t in (k_tree, v_tree, k_pool, v_pool)):
        raise TypeError("q, k_tree, v_tree and the pools must share one dtype out of float16, bfloat16")
    Z, H, n_q, D = q.shape
    H_kv = k_tree.shape[1]
    if k_tree.shape != (Z, H_kv, n_q, D) or v_tree.shape != k_tree.shape or H_kv < 1 or H % H_kv:
        raise ValueError("k_tree and v_tree must be [Z, H_kv, N, D] with H a multiple of H_kv")
    if pool_layout not in ("NHD", "HND"):
        raise ValueError("pool_layout must be 'NHD' or 'HND'")
    row_dim, head_dim_ = (1, 2) if pool_layout == "NHD" else (2, 1)
    n_pages, page_size = k_pool.shape[0], k_pool.shape[row_dim]
    if k_pool.dim() != 4 or v_pool.shape != k_pool.shape or k_pool.shape[head_dim_] != H_kv or k_pool.shape[3] != D \
            or k_pool.stride() != v_pool.stride() or k_pool.stride(3) != 1:
        raise ValueError("pools must be two equally laid out [n_pages, page_size, H_kv, D] (or HND) tensors")
    if block_table.dtype != torch.int32 or prefix_lens.dtype != torch.int32 or block_table.dim() != 2 \
            or block_table.shape[0] != Z or prefix_lens.shape != (Z,) or not block_table.is_contiguous():
        raise ValueError("block_table must be contiguous int32 [Z, pages], prefix_lens int32 [Z]")
    if meta.n_trees not in (1, Z) or meta.n_blocks != -(-n_q // meta.block_m):
        raise ValueError("metadata does not match q")
    if max_prefix is None:
        max_prefix = int(prefix_lens.max().item())
    if max_prefix <= 0:                                   # no prefix anywhere: plain tree attention
        return fst_attention(q, k_tree, v_tree, meta, sm_scale=sm_scale, out=out, return_lse=return_lse)
    o = torch.empty_like(q) if out is None else out
    if o.shape != q.shape or o.dtype != q.dtype or not o.is_cuda:
        raise ValueError("out must match q")
    lse = torch.empty((Z * H, n_q), device=q.device, dtype=torch.float32) if return_lse else None
    lib = _lib.lib()
    dev = q.device
    if kv_splits is None:
        sms = _SMS.get(dev)
        if sms is None:
            sms = _SMS[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
        ctas = Z * H * -(-n_q // 128)
        kv_splits = int(max(1, min(sms // max(ctas, 1), max_prefix // 256, 65535 // Z)))
    status = _status_record(dev)
    with _OnDevice(dev):
        ws_bytes = int(lib.fst_attention_split_workspace_bytes(Z, H, n_q, D, kv_splits))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        rc = lib.fst_attention_fwd_paged(
            q.data_ptr(), k_tree.data_ptr(), v_tree.data_ptr(), o.data_ptr(),
            lse.data_ptr() if lse is not None else None,
            meta.packed.data_ptr(), meta.tree_stride if meta.n_trees > 1 else 0,
            k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(), block_table.shape[1],
            prefix_lens.data_ptr(), int(max_prefix), page_size, n_pages,
            k_pool.stride(0), k_pool.stride(row_dim), k_pool.stride(head_dim_),
            Z, H, H_kv, n_q, D, *_strides(q), *_strides(k_tree), *_strides(v_tree), *_strides(o),
            meta.block_m, meta.max_ancestors, float(sm_scale), _DTYPES[q.dtype], kv_splits,
            ws.data_ptr(), ws_bytes, status.data_ptr(), _raw_stream(dev))
    _lib.check(rc, "fst_attention_fwd_paged")
    return (o, lse) if return_lse else o

