"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/mxdsa.h declares; the torch extension module loads and exposes the reference's two names."""
import ctypes
import os
import re

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "mxdsa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mxdsa_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_functions()
    for n in ("mxdsa_prefill_fwd", "mxdsa_decode_sched", "mxdsa_decode_fwd", "mxdsa_decode_workspace_bytes",
              "mxdsa_num_sm_parts", "mxdsa_status_string", "mxdsa_last_cuda_error", "mxdsa_device_fault"):
        assert n in names


def test_library_exports_every_declared_symbol():
    from mxdsa_b200 import capi
    lib = ctypes.CDLL(capi.LIB_PATH)
    for name in _declared_functions():
        assert hasattr(lib, name), name
    assert set(capi.EXPORTS) <= set(_declared_functions())


def test_status_strings_and_argument_checks_need_no_gpu():
    from mxdsa_b200 import capi
    L = capi.lib()
    assert L.mxdsa_status_string(0) == b"ok"
    assert b"NULL" in L.mxdsa_status_string(1)
    assert L.mxdsa_prefill_fwd(None) == 1          # MXDSA_ERR_NULL
    assert L.mxdsa_decode_fwd(None) == 1
    p = capi.PrefillParams(s_q=0, s_kv=4, topk=64, q=16, kv=16, indices=16, out=16, max_logits=16, lse=16)
    assert L.mxdsa_prefill_fwd(ctypes.byref(p)) == 2   # no query token -> MXDSA_ERR_SHAPE
    p = capi.PrefillParams(s_q=4, s_kv=4, topk=0, q=16, kv=16, indices=16, out=16, max_logits=16, lse=16)
    assert L.mxdsa_prefill_fwd(ctypes.byref(p)) == 2   # empty index rows
    p = capi.PrefillParams(s_q=3, s_kv=4, topk=96, q=16, kv=16, indices=16, out=16, max_logits=16, lse=16,
                           stride_q_token=64 * 528, stride_indices_pair=64)
    assert L.mxdsa_prefill_fwd(ctypes.byref(p)) == 2   # index rows closer together than topk
    p = capi.PrefillParams(s_q=4, s_kv=4, topk=64, q=24, kv=16, indices=16, out=16, max_logits=16, lse=16,
                           stride_q_token=64 * 528, stride_indices_pair=64)
    assert L.mxdsa_prefill_fwd(ctypes.byref(p)) == 3   # q not 16-byte aligned -> MXDSA_ERR_ALIGN
    assert L.mxdsa_decode_workspace_bytes(128, 6, 24) == (128 + 24) * 6 * 64 * 513 * 4
    assert L.mxdsa_decode_workspace_bytes(0, 6, 24) == 0
    # pack entry points: argument rules are checked before any CUDA call
    assert L.mxdsa_pack_q(None) == 1 and L.mxdsa_pack_kv(None) == 1
    q = capi.PackQParams(rows=0, src=16, src_dtype=capi.DTYPE_BF16, dst=16)
    assert L.mxdsa_pack_q(ctypes.byref(q)) == 0          # nothing to do
    q = capi.PackQParams(rows=2, src=16, src_dtype=7, dst=16)
    assert L.mxdsa_pack_q(ctypes.byref(q)) == 2          # unknown dtype
    q = capi.PackQParams(rows=2, src=24, src_dtype=capi.DTYPE_F32, dst=16)
    assert L.mxdsa_pack_q(ctypes.byref(q)) == 3          # source not 16-byte aligned
    q = capi.PackQParams(rows=2, src=16, src_dtype=capi.DTYPE_BF16, dst=16, dst_stride_row=520)
    assert L.mxdsa_pack_q(ctypes.byref(q)) == 3          # row stride below 528 / not a multiple of 16
    k = capi.PackKVParams(rows=10, src=16, src_dtype=capi.DTYPE_BF16, dst=16, rows_per_page=4)
    assert L.mxdsa_pack_kv(ctypes.byref(k)) == 2         # rows not a multiple of the page size
    k = capi.PackKVParams(rows=8, src=16, src_dtype=capi.DTYPE_BF16, dst=16, rows_per_page=0)
    assert L.mxdsa_pack_kv(ctypes.byref(k)) == 2
    # the combine step on its own keeps its per-warp weights in a fixed shared array of 192 splits
    c = capi.CombineParams(b=4, s_q=1, num_sm_parts=193, sched_meta=16, num_splits=16, workspace=32,
                           workspace_bytes=1 << 30, out=32, lse=16)
    assert L.mxdsa_decode_combine(ctypes.byref(c)) == 2   # more parts than the kernel can merge -> MXDSA_ERR_SHAPE


def test_extension_module_exposes_the_reference_entry_points():
    import mxdsa_b200
    ext = mxdsa_b200.ext()
    assert hasattr(ext, "dual_mxfp8_head64_sparse_prefill_fwd")
    assert hasattr(ext, "dual_mxfp8_sparse_decode_fwd")
    # the same file is importable under the reference's module name
    import importlib.util
    spec = importlib.util.spec_from_file_location("mxdsa_ext", mxdsa_b200._EXT_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert hasattr(mod, "dual_mxfp8_head64_sparse_prefill_fwd") and hasattr(mod, "dual_mxfp8_sparse_decode_fwd")


def test_topk_argument_checks_need_no_gpu():
    from mxdsa_b200 import capi
    L = capi.lib()
    assert L.mxdsa_topk_select(None) == 1
    ok = dict(scores=16, indices=16, rows=4, group=1, s_kv=16, topk=4)
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "scores": None}))) == 1
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "s_kv": 10}))) == 2     # not a multiple of 4
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "group": 3}))) == 2
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "topk": 0}))) == 2
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "scores": 20}))) == 3   # scores not 16-byte aligned
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "score_stride": 12}))) == 3   # stride below s_kv
    assert L.mxdsa_topk_select(ctypes.byref(capi.TopkParams(**{**ok, "rows": 0}))) == 0
