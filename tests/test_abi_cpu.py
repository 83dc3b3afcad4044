"""CPU: the C-ABI library builds, loads without a GPU driver and exports every symbol that
include/b200_attn.h declares; host-side argument checks that need no device."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("b200_store_kvcache", "b200_decode_attn", "b200_prefill_attn", "b200_decode_workspace_bytes",
                 "b200_last_error", "b200_version"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    from nanovllm_b200 import _lib
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in b200_attn.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(_declared())
    assert lib.b200_version() == 100


def test_binding_arity_matches_header():
    from nanovllm_b200 import _lib
    text = open(os.path.join(ROOT, "include", "b200_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, (_, args) in _lib.SIGNATURES.items():
        m = re.search(r"\b%s\s*\(([^)]*)\)" % name, text)
        params = m.group(1).strip()
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(args), name


def test_host_side_rejections_need_no_device(lib):
    assert lib.b200_store_kvcache(None, None, 0, 0, None, None, None, 0, 1024, 2, 0, None) == 0   # empty: no-op
    assert lib.b200_store_kvcache(None, None, 0, 0, None, None, None, 4, 1024, 2, 10, None) == -1
    assert b"null" in lib.b200_last_error()
    assert lib.b200_store_kvcache(16, 16, 1024, 1024, 16, 16, 16, 4, 1023, 2, 10, None) == -3
    assert lib.b200_store_kvcache(16, 16, 1024, 1024, 16, 16, 16, -1, 1024, 2, 10, None) == -2
    assert lib.b200_decode_attn(16, 2048, 16, 16, 1, 256, 16, 1, 1, 16, 16, 16, 1 << 30, 0, 16, 8, 128, 0.1, None) == 0
    assert lib.b200_decode_attn(16, 2048, 16, 16, 1, 256, 16, 1, 1, 16, 16, 16, 1 << 30, 1, 16, 8, 96, 0.1, None) == -2
    assert lib.b200_decode_attn(16, 2048, 16, 16, 1, 300, 16, 1, 1, 16, 16, 16, 1 << 30, 1, 16, 8, 128, 0.1, None) == -2
    assert lib.b200_decode_attn(16, 2048, 16, 16, 1, 256, 16, 1, 1, 16, 16, 16, 1 << 30, 1, 16, 5, 128, 0.1, None) == -2
    assert lib.b200_decode_attn(18, 2048, 16, 16, 1, 256, 16, 1, 1, 16, 16, 16, 1 << 30, 1, 16, 8, 128, 0.1, None) == -3
    assert lib.b200_prefill_attn(16, 2048, 16, 16, 1024, 1024, 8, None, None, 0, 0, None, 0, 0, 16, 16, 1, 8, 8, 8, 16,
                                 16, 8, 64, 0.1, 0, None) == -2
    assert lib.b200_decode_workspace_bytes(0, 16, 8, 128) == -2


def test_no_cpu_fallback_in_the_product():
    import nanovllm_b200
    q = torch.zeros(1, 16, 128, dtype=torch.bfloat16)
    c = torch.zeros(1, 256, 8, 128, dtype=torch.bfloat16)
    i = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nanovllm_b200.decode_attention(q, c, c, i, i.view(1, 1), 0.1, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nanovllm_b200.store_kvcache(torch.zeros(1, 8, 128, dtype=torch.bfloat16), torch.zeros(1, 8, 128, dtype=torch.bfloat16), c, c, i)


def test_product_does_not_import_the_oracle():
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); import nanovllm_b200, nanovllm_b200.integration, nanovllm_b200.sharding; "
            "bad = [m for m in sys.modules if m.startswith('oracle') or m.startswith('flash_attn') or m == 'triton']; "
            "print(bad); sys.exit(1 if bad else 0)") % ROOT
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
