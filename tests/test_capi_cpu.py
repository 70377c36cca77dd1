"""The C-ABI library builds, loads and exports every symbol the header declares;
argument validation answers with error codes (no GPU needed, no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "axp_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(axp_sm100_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib(pkg):
    pkg.capi.build()
    return pkg.capi.lib()


def test_header_symbols_all_exported(lib, pkg):
    names = declared_symbols()
    assert set(names) == set(pkg.capi.EXPORTS)
    for n in names:
        assert getattr(lib, n) is not None


def test_fnv1a64_matches_reference_definition(pkg, lib):
    def fnv(s):
        h = 14695981039346656037
        for ch in s.encode():
            h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        return h

    for s in ("", "a", "preset.gemm.fp8bs.128x256x128", "axp.l4.profile.proof_full"):
        assert pkg.capi.fnv1a64(s) == fnv(s)


def test_query_known_and_unknown_keys(pkg, lib):
    caps = pkg.capi.query("preset.gemm.fp8bs.128x256x128")
    assert (caps.op_family, caps.elem_bits, caps.tile_m, caps.tile_n, caps.tile_k) == (1, 8, 128, 256, 128)
    assert caps.tmem_columns == 512 and caps.smem_bytes <= 227 * 1024
    caps = pkg.capi.query("preset.attention.bf16.128x128x128.causal")
    assert caps.op_family == 2 and caps.elem_bits == 16
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.capi.query("preset.sort.16")          # the reference keeps sort unsupported on sm100
    assert e.value.code == pkg.capi.AXP_ERR_UNSUPPORTED


def test_bad_arguments_return_codes_without_touching_a_gpu(pkg, lib):
    z = ctypes.c_void_p(0)
    p = ctypes.c_void_p(4096)      # never dereferenced: validation fails first
    rc = lib.axp_sm100_gemm_bf16(z, p, p, 128, 128, 128, 128, 128, 128, 0, 128, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG and b"null" in lib.axp_sm100_last_error()
    rc = lib.axp_sm100_gemm_fp8_blockscaled(p, p, p, p, p, 128, 256, 200, 256, 256, 256, 0, 256, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG and b"128" in lib.axp_sm100_last_error()      # K % 128
    rc = lib.axp_sm100_gemm_fp8_blockscaled(p, p, p, p, p, 128, 256, 256, 256, 256, 256, 64, 256, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG                                               # n_begin % 128
    rc = lib.axp_sm100_gemm_bf16(p, p, p, 128, 128, 128, 128, 128, 128, 0, 256, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG                                               # n_end > N
    rc = lib.axp_sm100_gemm_bf16(ctypes.c_void_p(4100), p, p, 128, 128, 128, 128, 128, 128, 0, 128, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG                                               # misaligned base
    # a column range that does not span a multiple of 8 columns would let the 8-wide epilogue stores run into the
    # neighbouring shard: rejected by every GEMM entry point
    rc = lib.axp_sm100_gemm_bf16(p, p, p, 128, 256, 128, 128, 128, 256, 0, 100, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG and b"multiple of 8" in lib.axp_sm100_last_error()
    rc = lib.axp_sm100_gemm_fp8_blockscaled(p, p, p, p, p, 128, 256, 256, 256, 256, 256, 128, 228, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG and b"multiple of 8" in lib.axp_sm100_last_error()
    rc = lib.axp_sm100_gemm_bf16_swiglu(p, p, p, p, 128, 256, 128, 128, 128, 128, 256, 0, 100, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG and b"multiple of 8" in lib.axp_sm100_last_error()
    rc = lib.axp_sm100_gemm_fp8_blockscaled_swiglu(p, p, p, p, p, p, p, 128, 256, 256, 256, 256, 256, 256, 0, 100, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG and b"multiple of 8" in lib.axp_sm100_last_error()
    rc = lib.axp_sm100_attn_fwd_bf16(p, p, p, p, z, 1, 4, 3, 128, 128, ctypes.c_float(1.0), 1, 0, 4, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG                                               # Hq % Hkv
    rc = lib.axp_sm100_attn_fwd_bf16(p, p, p, p, z, 1, 4, 4, 128, 64, ctypes.c_float(1.0), 1, 0, 4, z, z)
    assert rc == pkg.capi.AXP_ERR_UNSUPPORTED                                           # head dim != 128
    rc = lib.axp_sm100_selftest_bounded_wait(0, z, z)
    assert rc == pkg.capi.AXP_ERR_BAD_ARG


def test_ops_refuse_cpu_tensors(pkg):
    import torch

    a = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        pkg.ops.gemm_bf16(a, a)


def test_missing_library_fails_loudly(pkg, monkeypatch):
    monkeypatch.setattr(pkg.capi, "_lib", None)
    monkeypatch.setattr(pkg.capi, "LIB_PATH", "/nonexistent/libaxp_sm100.so")
    with pytest.raises(FileNotFoundError):
        pkg.capi.lib()
