"""Host-side checks that need no GPU: the C-ABI library builds, loads and exports every symbol
the header declares; argument validation returns error codes before anything is launched; the
Python mirror raises where the reference asserts; workspace sizing."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(built_library):
    from vecattention_b200 import _lib
    return _lib


def test_header_symbols_are_exported(lib):
    header = open(os.path.join(ROOT, "include", "vecattn.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(va_\w+)\s*\(", header, flags=re.M))
    assert declared == set(lib.EXPORTS), declared ^ set(lib.EXPORTS)
    handle = lib.lib()
    for name in declared:
        assert hasattr(handle, name)
    assert handle.va_version() >= 200
    assert lib.status_string(0) == "ok"
    for code in range(-8, 0):
        assert "unknown" not in lib.status_string(code)


def test_struct_layout_matches_header(lib):
    # sizes of the C structs as the compiler lays them out (LP64): guards against drift between
    # include/vecattn.h and the ctypes mirror
    assert C.sizeof(lib.Tensor4) == 32
    assert C.sizeof(lib.PoolArgs) == 24 + 32 + 8
    assert C.sizeof(lib.SelectArgs) == 56 + 8 + 32 + 8 + 8 + 8 + 8 + 8 + 8 + 8 + 8 + 8 + 8
    assert C.sizeof(lib.AttnArgs) == 40 + 4 * 32 + 8 * 6 + 8 + 8 + 8 + 16   # ... + three int32 and padding
    assert C.sizeof(lib.NormRopeArgs) == 24 + 8 * 8 + 8 * 2 + 8 + 8 + 8
    assert C.sizeof(lib.HeadNormRopeArgs) == 24 + 4 * 32 + 8 * 2 + 8 + 8 * 2
    assert C.sizeof(lib.PrefillArgs) == 56 + 4 * 32 + 8 + 8 + 8 + 8 + 8 + 8 + 8 + 8


def test_validation_returns_codes_without_launching(lib):
    h = lib.lib()
    assert h.va_pool_q(None, None) == -1
    assert h.va_select(None, None) == -1
    assert h.va_sparse_attn(None, None) == -1
    assert h.va_prefill(None, None) == -1
    a = lib.PoolArgs(7, 1, 1, 64, 128, 64, lib.Tensor4(16, 0, 0, 128), 16)
    assert h.va_pool_q(C.byref(a), None) == -2          # dtype
    a.dtype = 0
    a.head_dim = 64
    assert h.va_pool_q(C.byref(a), None) == -3          # head_dim
    a.head_dim = 128
    a.pq = 32
    assert h.va_pool_q(C.byref(a), None) == -7          # q_pooling_size
    a.pq = 64
    a.q.ptr = 8
    assert h.va_pool_q(C.byref(a), None) == -4          # alignment
    s = lib.SelectArgs()
    s.avg_q, s.col_count, s.col_idx = 16, 16, 16
    s.dtype, s.batch, s.heads, s.kv_heads, s.nq, s.sk, s.head_dim = 0, 1, 3, 2, 4, 256, 128
    s.pq, s.bk, s.group_k_block, s.capacity = 64, 16, 1, 256
    assert h.va_select(C.byref(s), None) == -3          # heads % kv_heads
    s.heads = 4
    s.bk = 24
    assert h.va_select(C.byref(s), None) == -3          # k_local_size
    s.bk = 128
    s.causal = 1
    assert h.va_select(C.byref(s), None) == -7          # causal needs pq % bk == 0
    s.bk, s.capacity = 16, 0
    assert h.va_select(C.byref(s), None) == -5          # capacity
    assert h.va_block_tables(1, 1, 128, 64, 1, None, None, None) == -1
    # vision-slice composition: 64-row tiles, causal, one sequence for queries and keys, ordered positions
    t = lib.Tensor4(256, 0, 0, 128)
    at = lib.AttnArgs(0, 1, 2, 2, 512, 512, 128, 64, 1, 0, t, t, t, t, None, None, 0, 256, 256, 16, 0.0, None, None, 1, 100, 400)
    at.pq = 128
    assert h.va_sparse_attn(C.byref(at), None) == -7
    at.pq, at.causal = 64, 0
    assert h.va_sparse_attn(C.byref(at), None) == -7
    at.causal, at.sk = 1, 1024
    assert h.va_sparse_attn(C.byref(at), None) == -7
    at.sk, at.vision_begin = 512, 401
    assert h.va_sparse_attn(C.byref(at), None) == -3
    at.vision_begin, at.vision_end = 100, 513
    assert h.va_sparse_attn(C.byref(at), None) == -3


def test_prefill_workspace_bytes(lib):
    h = lib.lib()
    a = lib.PrefillArgs()
    a.dtype, a.batch, a.heads, a.kv_heads, a.sq, a.sk, a.head_dim = 0, 1, 32, 32, 32768, 32768, 128
    a.pq, a.bk, a.group_k_block, a.causal, a.chunk_size, a.compat_bsq = 64, 16, 16, 0, 32768, 64
    n = C.c_size_t(0)
    assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(n)) == 0
    idx_bytes = 32 * 512 * 32768 * 4
    mask_bytes = 32 * 512 * (32768 // 32) * 4          # one keep bit per (pooled row, key)
    assert idx_bytes + mask_bytes <= n.value <= idx_bytes + mask_bytes + 8 * 2 ** 20
    # the whole sequence fits the single-pass budget: chunk_size does not change the workspace
    a.chunk_size = 8192
    n2 = C.c_size_t(0)
    assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(n2)) == 0
    assert n2.value == n.value
    # a sequence whose index lists exceed the budget: chunk_size bounds the workspace as in the reference
    a.heads = a.kv_heads = 64
    a.sq = a.sk = 262144
    a.chunk_size = 32768
    big = C.c_size_t(0)
    assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(big)) == 0
    assert 64 * 512 * 262144 * 4 <= big.value <= 64 * 512 * 262144 * (4 + 1 / 8) + 64 * 2 ** 20
    a.chunk_size = 8192
    small = C.c_size_t(0)
    assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(small)) == 0
    assert small.value < big.value / 3.9
    # the budget belongs to the caller: the quick-use shape (2 GiB of index lists) goes through the chunk
    # loop once the budget is below that, and the workspace then shrinks with chunk_size
    a.heads = a.kv_heads = 32
    a.sq = a.sk = 32768
    sizes = []
    for budget, chunk in [(0, 8192), (1 << 30, 32768), (1 << 30, 8192), (1, 4096)]:
        a.single_pass_budget, a.chunk_size = budget, chunk
        assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(n2)) == 0
        sizes.append(n2.value)
    assert sizes[0] == n.value and sizes[1] == n.value      # one chunk covers the sequence
    assert sizes[2] < n.value / 3.9 and sizes[3] < n.value / 7.5
    a.single_pass_budget = 0
    a.chunk_size = 100
    assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(n2)) == -7
    a.chunk_size, a.causal, a.sk = 8192, 1, 4096
    assert h.va_prefill_workspace_bytes(C.byref(a), C.byref(n2)) == -7   # causal needs Sq == Sk
    a.causal, a.workspace, a.workspace_bytes = 0, 256, 1024
    a.q = a.k = a.v = a.out = lib.Tensor4(256, 0, 0, 128)
    assert h.va_prefill(C.byref(a), None) == -5                           # workspace too small


def test_python_mirror_raises_like_the_reference(built_library):
    import vecattention_b200 as va
    q = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        va.VecAttention_prefill(q, q, q, 0.5, 64, 16, 16, False, chunk_size=100)
    with pytest.raises(AssertionError):
        va.VecAttention_prefill(q, q, q, 0.5, 32, 16, 16, False, chunk_size=1024)
    with pytest.raises(TypeError):
        va.VecAttention_prefill(q, q, q, None, 64, 16, 16, False, chunk_size=1024)
    # no CPU fallback: host tensors are refused, loudly
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        va.VecAttention_prefill(q, q, q, 0.5, 64, 16, 16, False, chunk_size=1024)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        va.average_vector(q, 64)


def test_missing_library_fails_loudly(monkeypatch, built_library):
    from vecattention_b200 import _lib
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libvecattn.so")
    with pytest.raises(RuntimeError, match="missing"):
        _lib.lib()


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "vecattention_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("CPU oracle uses the same association", ""), f


def test_host_pipeline_slices_cover_whole_kv_groups(built_library):
    from vecattention_b200.hostio import head_slices, transfer_bytes
    for heads, kv, n in [(32, 32, 8), (28, 4, 8), (12, 4, 5), (8, 8, 1), (6, 2, 3)]:
        parts = head_slices(heads, kv, n)
        rep = heads // kv
        assert parts[0][0] == 0 and parts[-1][1] == heads
        assert all(a1 == b0 for (_, a1), (b0, _) in zip(parts, parts[1:]))
        assert all((h1 - h0) % rep == 0 and h1 > h0 for h0, h1 in parts)
        assert len(parts) == min(n, kv)
    assert transfer_bytes(1, 32, 32, 32768, 32768, 128, 2) == (805306368, 268435456)


def test_host_pipeline_fails_loudly_without_a_gpu(built_library):
    import torch
    from vecattention_b200.hostio import VecAttention_prefill_host
    if torch.cuda.is_available():
        pytest.skip("needs a box without a GPU")
    q = torch.zeros(1, 2, 64, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        VecAttention_prefill_host(q, q, q, 0.5, 64, 16, 16, False, 64)


def test_dense_block_tables_cover_keys_up_to_the_diagonal(built_library):
    import torch
    from vecattention_b200.vision import dense_block_tables
    for row0, rows in [(0, 64), (37, 100), (1900, 148), (0, 1), (63, 2), (128, 640)]:
        cnt, start = dense_block_tables(2, 3, row0, rows, "cpu")
        nq = -(-rows // 64)
        assert cnt.shape == (2, 3, nq) and start.shape[:3] == (2, 3, nq) and cnt.dtype == torch.int32
        for t in range(nq):
            last = min(row0 + 64 * (t + 1), row0 + rows) - 1
            n = int(cnt[1, 2, t])
            assert n == last // 64 + 1 and n <= start.shape[3]
            assert start[1, 2, t, :n].tolist() == [64 * i for i in range(n)]


def test_threshold_files_and_guidance_switch(tmp_path, built_library):
    import torch
    from vecattention_b200.thresholds import GuidanceThresholds, load_threshold_matrix, save_threshold_matrix
    path = str(tmp_path / "thr.json")
    mat = torch.rand(3, 4)
    save_threshold_matrix(path, mat, 3, 4)
    back = load_threshold_matrix(path, 3, 4)
    assert back.dtype == torch.float32 and back.is_contiguous() and torch.allclose(back, mat)
    save_threshold_matrix(path, 0.5, 2, 5)
    assert load_threshold_matrix(path, 2, 5).eq(0.5).all()
    for layers, heads in [(3, 5), (2, 4)]:  # wrong shape on either axis
        with pytest.raises(RuntimeError, match="Cannot load threshold file"):
            load_threshold_matrix(path, layers, heads)
    with pytest.raises(RuntimeError):
        load_threshold_matrix(str(tmp_path / "missing.json"), 1, 1)
    # two passes per diffusion step: positive first, negative on the repeated timestep
    pos, neg = torch.full((2, 4), 0.9), torch.full((2, 4), 0.6)
    g = GuidanceThresholds(pos, neg)
    picks = [g.select(t) is pos for t in (999.0, 999.0, 950.0, 950.0, 900.0)]
    assert picks == [True, False, True, False, True] and g.step == 3
    assert g.for_layer(1).shape == (4,) and g.for_layer(1).eq(0.9).all()
    assert GuidanceThresholds(0.7, guidance=False).select(1.0) == 0.7


def test_stage_workspace_queries(lib):
    import ctypes as C
    # selection: one keep bit per (pooled row, key), rows in CTAs of 128, keys in groups of four 128-key tiles
    a = lib.SelectArgs()
    a.batch, a.heads, a.kv_heads, a.nq, a.sk = 1, 40, 40, 1182, 75600
    n = C.c_size_t(0)
    assert lib.lib().va_select_workspace_bytes(C.byref(a), C.byref(n)) == 0
    assert n.value == 40 * 1280 * (148 * 16) * 4
    a.heads, a.kv_heads, a.nq, a.sk = 28, 4, 1024, 65536       # 7 query heads share the rows of one KV head
    assert lib.lib().va_select_workspace_bytes(C.byref(a), C.byref(n)) == 0
    assert n.value == 4 * 7168 * 2048 * 4
    a.heads = 27
    assert lib.lib().va_select_workspace_bytes(C.byref(a), C.byref(n)) == -3
    # a selection without its scratch is refused before anything is launched
    s = lib.SelectArgs()
    s.avg_q, s.col_count, s.col_idx = 16, 16, 16
    s.dtype, s.batch, s.heads, s.kv_heads, s.nq, s.sk, s.head_dim = 0, 1, 4, 2, 4, 256, 128
    s.pq, s.bk, s.group_k_block, s.capacity = 64, 16, 1, 256
    s.k = lib.Tensor4(256, 0, 0, 128)
    assert lib.lib().va_select(C.byref(s), None) == -1
    s.workspace, s.workspace_bytes = 256, 16
    assert lib.lib().va_select(C.byref(s), None) == -5
    n = C.c_size_t(123)
    assert lib.lib().va_sparse_attn_workspace_bytes(C.byref(lib.AttnArgs()), C.byref(n)) == 0 and n.value == 0
    assert lib.lib().va_select_workspace_bytes(None, C.byref(n)) == -1


def test_fastprefill_config_and_flags(built_library):
    """The caller-side configuration object and its command-line flags, with the reference's names and
    defaults (spattn/src/models/config_args.py)."""
    import argparse
    from vecattention_b200 import (FastPrefillConfig, add_fastprefill_args, build_output_file_from_config,
                                   get_fastprefill_config)
    c = FastPrefillConfig()
    assert (c.metric, c.block_size_q, c.block_size_k, c.group_k_block, c.chunk_size) == ("xattn", 64, 16, 1, 8192)
    assert c.vision_start_position is None and c.output_time is True and c.input_id == "input"
    assert not hasattr(c, "threshold") and "threshold" not in c       # only present when given
    c = FastPrefillConfig(metric="vecattention", threshold=0.8, group_k_block=16)
    assert c.threshold == 0.8 and c["group_k_block"] == 16 and isinstance(c, dict)
    c.vision_end_position = 100
    assert c["vision_end_position"] == 100
    with pytest.raises(TypeError):
        FastPrefillConfig(no_such_field=1)
    ap = add_fastprefill_args(argparse.ArgumentParser())
    ns = ap.parse_args([])
    assert (ns.fastprefill_metric, ns.fastprefill_threshold, ns.fastprefill_chunk_size) == ("full", 0.9, 65536)
    ns = ap.parse_args("--fastprefill-metric vecattention --fastprefill-threshold 0.7 --fastprefill-group-k-block 8192 "
                       "--fastprefill-block-size-k 16 --fastprefill-chunk-size 32768".split())
    c = get_fastprefill_config(ns)
    assert (c.metric, c.threshold, c.group_k_block, c.chunk_size, c.input_id) == ("vecattention", 0.7, 8192, 32768, "input")
    assert build_output_file_from_config("out/res.json", c) == "out/res_metric=vecattention_th=0.7_qps=64_kls=16_gkb=8192.json"
    assert build_output_file_from_config("r.txt", FastPrefillConfig(metric="full")) == "r_metric=full.txt"
