"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _built():
    from statetree_b200 import ops
    if not os.path.exists(ops.LIB_PATH):
        import importlib.util
        spec = importlib.util.spec_from_file_location("st_build", os.path.join(ROOT, "statetree-representation_b200",
                                                                               "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_library()
    return ops


def test_library_exports_header_symbols():
    ops = _built()
    with open(os.path.join(ROOT, "include", "statetree_b200.h")) as f:
        text = f.read()
    declared = set(re.findall(r"\b(st_[a-z0-9_]+)\s*\(", text))
    assert declared == set(ops.exported_symbols()), declared ^ set(ops.exported_symbols())
    L = ops.lib()                                       # resolves every symbol, checks the ABI version
    assert L.st_abi_version() == ops.ABI
    assert L.st_kv_page_bytes(1) == 6400 and L.st_kv_page_bytes(8) == 51200


def test_argument_errors_are_reported_without_a_gpu():
    ops = _built()
    L = ops.lib()
    assert L.st_dec(None, None, None, 17, 64, None, None) != 0
    assert b"M % 16" in L.st_last_error()
    assert L.st_gemv(None, None, None, None, None, None, None, 33, 16, 64, None, 0, None, None) != 0
    assert b"batch" in L.st_last_error()
    assert L.st_gemm(None, None, None, None, None, None, 64, 64, 64, None, 0, None, None) != 0
    assert L.st_gemv_workspace_bytes(100, 64, 1) == -1
    # the exchange entry points check rank / world and sizes before anything touches a GPU
    assert L.st_comm_bytes() == 8 * 64 * 4 + 64 * 4 + 256 + 2 * 8 * 64 * 16384 + 2 * 8 * (128 << 10) * 4
    assert L.st_gemv_allreduce(None, 0, 9, None, None, None, None, None, None, None, 1, 64, 64, None, 0, None) != 0
    assert b"ranks" in L.st_last_error()
    assert L.st_gemm_list(0, None, None, None, None, None, None, 1, None, 64, None, None) != 0
    assert L.st_gemv_list(5, None, None, None, None, None, None, None, 1, None, 64, None, 0, None) != 0
    assert b"1 to 4" in L.st_last_error()
    assert L.st_comm_set_timeout_ms(0) != 0
    assert L.st_allreduce(None, 0, 1, None, None, 8, None) != 0
    assert b"ranks" in L.st_last_error()
    assert L.st_allreduce_add_rmsnorm(None, 3, 2, None, None, None, None, 1, 4096, 1e-6, None) != 0
    assert L.st_moe_align(None, 1, 0, 8, 8, 8, None, None, None, 4, None) != 0
    assert L.st_moe_align(None, 1, 8, 2048, 2048, 8, None, None, None, 16, None) != 0 and b"experts" in L.st_last_error()
    assert L.st_moe_group_gemm(None, None, None, 4, None, None, None, None, 4, 32, None, None, 8, 128, 64, None) != 0
    assert b"block size" in L.st_last_error()


def test_cpu_tensors_are_rejected():
    import torch
    ops = _built()
    with pytest.raises(RuntimeError):
        ops.ext().dec(torch.zeros(1, 1, 1552, dtype=torch.uint8), torch.zeros(2, dtype=torch.int32),
                      torch.zeros(1, dtype=torch.int32), torch.zeros(16, 64, dtype=torch.bfloat16))


def test_package_exports_the_reference_names():
    """`import statetree_b200 as statetree` keeps a caller's lines: the names statetree/__init__.py:10-17 exports"""
    import statetree_b200 as S
    names = ["TreeLinear", "TreeSlice", "TreeEmbedding", "TreeExperts", "DEFAULT_FUSE", "convert", "prepare",
             "save_pretrained", "load_pretrained", "size_report", "tree_modules", "encode", "decode_reference"]
    assert sorted(S.__all__) == sorted(names)
    for n in names:
        assert hasattr(S, n), n
    assert S.DEFAULT_FUSE["qkv_proj"] == ("q_proj", "k_proj", "v_proj")


def test_install_as_makes_the_reference_imports_resolve_here():
    import importlib
    import sys
    import statetree_b200 as S
    try:
        S.install_as("statetree_alias_for_test")
        import statetree_alias_for_test as A                      # noqa: F401
        from statetree_alias_for_test.linear import TreeLinear
        assert A is S and TreeLinear is S.TreeLinear
        assert importlib.import_module("statetree_alias_for_test.ops").ext is S.ops.ext
        assert importlib.import_module("statetree_alias_for_test._vllm").StateTreeLinearMethod is not None
        sys.modules["taken_name_for_test"] = sys
        with pytest.raises(RuntimeError, match="already imported"):
            S.install_as("taken_name_for_test")
    finally:
        for k in [k for k in sys.modules if k.startswith("statetree_alias_for_test") or k == "taken_name_for_test"]:
            del sys.modules[k]
