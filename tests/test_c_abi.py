"""The shared library loads and exports every symbol the public header declares (no GPU needed)."""

import ctypes
import re
from pathlib import Path

import pytest

from kestrel_b200 import _native, kernels

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "kestrel_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"KB200_API[^;(]*?\b(kb200_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_symbols()
    assert len(names) >= 9
    assert sorted(_native.EXPORTS) == names


def test_library_exports_every_declared_symbol():
    lib = _native.load()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.kb200_abi_version() == _native.ABI_VERSION


def test_struct_layout_matches_header_field_order():
    text = HEADER.read_text()
    body = text[text.index("typedef struct kb200_attn_args"):text.index("} kb200_attn_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        for part in decl.split(","):
            fields.append(re.findall(r"(\w+)\s*$", part.strip())[0])
    assert fields == [f[0] for f in _native.AttnArgs._fields_]
    assert ctypes.sizeof(_native.AttnArgs) % 8 == 0


def test_argument_errors_surface_without_a_gpu():
    lib = _native.load()
    assert lib.kb200_attn_workspace_bytes(0, 0, 0, 0, 0, 0) == 0
    rc = lib.kb200_paged_attention(None)
    assert rc == -1
    assert b"null" in lib.kb200_last_error()
    with pytest.raises(ValueError):
        _native.check(rc)


def test_runtime_object_has_the_reference_entry_points():
    rt = kernels.get_runtime()
    assert callable(rt.cache.reshape_and_cache_flash)
    assert callable(rt.cache.build_paged_kv_metadata)
    assert callable(rt.attention.flash_attn_fwd)
    assert callable(rt.sampling.sample_step_from_logits)
    with pytest.raises(NotImplementedError):
        rt.moe.topk_fwd
    assert rt.attention.block_bidirectional_mask is kernels.block_bidirectional_mask
    with pytest.raises(NotImplementedError):
        rt.attention.flash_attn_varlen_func


def test_cpu_tensors_are_rejected_loudly():
    import torch

    k = torch.zeros(1, 2, 8)
    cache = torch.zeros(2, 4, 2, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        kernels.reshape_and_cache_flash(k, k, cache, cache, torch.zeros(1, dtype=torch.int64), "auto", None, None)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        kernels.flash_attn_fwd(torch.zeros(1, 1, 2, 8, dtype=torch.bfloat16), cache, cache,
                               page_table=torch.zeros(1, 1, dtype=torch.int32),
                               seqused_k=torch.ones(1, dtype=torch.int32))
    with pytest.raises(NotImplementedError):
        kernels.flash_attn_fwd(torch.zeros(1, 1, 2, 8), cache, cache)


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_native.NativeLibraryError, match="no CPU or PyTorch fallback"):
        _native.load()
