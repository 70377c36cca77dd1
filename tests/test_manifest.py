"""Manifest rows, generated registry index, compile-time resolution and the launch
shim's dispatch table agree with each other (CPU only)."""
import copy
import importlib
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tool():
    return importlib.import_module("iro-cuda-ax_b200.manifest_tool")


def test_manifest_validates(tool):
    assert tool.validate(tool.load()) == []


def test_registry_index_is_up_to_date(tool):
    assert open(tool.INDEX).read() == tool.render_index(tool.load())


def test_validator_rejects_broken_rows(tool):
    doc = tool.load()
    def bad(mut):
        d = copy.deepcopy(doc)
        mut(d)
        return tool.validate(d)
    assert bad(lambda d: d["kernels"].reverse())                                   # not sorted by id
    assert bad(lambda d: d["kernels"][0].pop("config"))                            # missing key
    assert bad(lambda d: d["kernels"][0].update(extra=1))                          # extra key
    assert bad(lambda d: d["kernels"][0].update(pattern="my::Pattern"))            # not a canonical preset
    assert bad(lambda d: d["kernels"][0].update(graph_hash="0x15583dd84da2d8e9"))  # reference hash reused
    assert bad(lambda d: d["kernels"][0].update(capability="sm90"))                # wrong lane
    assert bad(lambda d: d["kernels"][1].update(realization_key=d["kernels"][0]["realization_key"]))
    assert bad(lambda d: d.update(schema_version=1))


def test_rows_match_the_shim_dispatch_table(tool, pkg):
    pkg.capi.build()
    for row in tool.load()["kernels"]:
        caps = pkg.capi.query(row["realization_key"])
        cfg = row["config"]
        assert caps.realization_key == tool.fnv1a64(row["realization_key"])
        assert [caps.tile_m, caps.tile_n, caps.tile_k] == cfg["tile"]
        assert caps.op_family == {"gemm": 1, "attention": 2, "gemm_fused": 3}[row["op_family"]]
        assert caps.elem_bits == {"bf16": 16, "e4m3": 8}[cfg["dtype"]]
        assert caps.tmem_columns == cfg["tmem_columns"] and caps.threads == cfg["threads"]
        assert caps.stages == cfg.get("stages", cfg.get("kv_stages"))
        assert caps.smem_bytes == cfg["smem_bytes"] and caps.cta_group == cfg["cta_group"]
        assert 0 < caps.smem_bytes <= 227 * 1024
        assert cfg["entry_point"] in pkg.capi.EXPORTS
        assert hasattr(pkg.capi.lib(), cfg["entry_point"])
        assert os.path.exists(os.path.join(ROOT, cfg["evidence"])), "each row names its committed ncu summary"


def test_compile_time_resolution_of_every_row():
    out = subprocess.run(["bash", os.path.join(ROOT, "tests", "compile", "check_sm100_rows.sh")],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


def test_generated_instantiation_units_compile_for_both_profiles(tmp_path):
    """`gen-instantiations --compile`: one translation unit per (row, profile); declared pairs resolve with their
    hash and key and bind every obligation, undeclared pairs are unsupported (the reference's generated TUs +
    scripts/compile.sh)."""
    import sys

    tool = os.path.join(ROOT, "iro-cuda-ax_b200", "manifest_tool.py")
    out = subprocess.run([sys.executable, tool, "gen-instantiations", "--out", str(tmp_path), "--compile"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    rows = json.load(open(os.path.join(ROOT, "manifests", "kernels_sm100.json")))["kernels"]
    units = sorted(p for p in os.listdir(tmp_path) if p.endswith(".cu"))
    assert len(units) == 2 * len(rows)
    assert out.stdout.count("ok   ") == len(units) and "FAIL" not in out.stdout
    # a unit whose declared hash is wrong must not compile
    bad = tmp_path / "bad.cu"
    good = (tmp_path / f"inst_{rows[0]['id']}__proof_full.cu").read_text()
    bad.write_text(good.replace(rows[0]["graph_hash"], "0x1"))
    r = subprocess.run(["/usr/local/cuda/bin/nvcc", "-std=c++20", "-ccbin", "/usr/bin/g++", "-gencode", "arch=compute_100a,code=sm_100a",
                        "-Wno-deprecated-gpu-targets", "-I" + os.path.join(ROOT, "include"), "-c", str(bad), "-o", str(tmp_path / "bad.o")],
                       capture_output=True, text=True)
    assert r.returncode != 0 and "declared graph hash" in r.stderr


def test_query_answers_from_the_configuration_the_kernels_are_checked_against(pkg):
    """`axp_sm100_query` is filled from csrc/kernel_config.hpp, which the kernel translation units static_assert their own
    constants against and tests/compile/sm100_rows.cu compares with the level-3 graphs: the header's numbers, parsed here as
    text, are what the library answers."""
    import re

    text = open(os.path.join(ROOT, "iro-cuda-ax_b200", "csrc", "kernel_config.hpp")).read()

    def ints(name):
        body = re.search(name + r"\s*=\s*\{([^}]*)\}", text).group(1)
        return [int(eval(x.replace("true", "1").replace("false", "0"))) for x in body.split(",")]

    pkg.capi.build()
    for key, name in (("preset.gemm.fp8bs.128x256x128", "kGemmFp8"), ("preset.gemm.bf16.128x256x64", "kGemmBf16")):
        tile_m, tile_n, tile_k, cta_group, stages, _, dyn_smem, tmem, threads, _, _ = ints(name)
        c = pkg.capi.query(key)
        assert (c.tile_m, c.tile_n, c.tile_k, c.cta_group, c.stages, c.smem_bytes, c.tmem_columns, c.threads) == \
            (tile_m, tile_n, tile_k, cta_group, stages, dyn_smem, tmem, threads)
    for key, name in (("preset.attention.bf16.128x128x128.causal", "kAttnBf16"), ("preset.attention.fp8.gqa.128x128x128.causal", "kAttnFp8")):
        tile_q, kv_tile, head_dim, _, kv_stages, dyn_smem, tmem, threads, _, _, _, _ = ints(name)
        c = pkg.capi.query(key)
        assert (c.tile_m, c.tile_n, c.tile_k, c.stages, c.smem_bytes, c.tmem_columns, c.threads) == \
            (tile_q, kv_tile, head_dim, kv_stages, dyn_smem, tmem, threads)


@pytest.mark.skipif(not os.environ.get("AXP_REFERENCE_CHECKOUT"), reason="set AXP_REFERENCE_CHECKOUT to a checkout of the reference project")
def test_reference_manifest_tool_accepts_the_sm100_rows(tmp_path):
    """The reference's own tool (tools/ax_manifest_tool.cpp, built here with g++) validates manifests/kernels_sm100.json
    together with its sm89 / sm90 manifests: the rows are a drop-in for the reference's empty sm100 manifest."""
    ref = os.environ["AXP_REFERENCE_CHECKOUT"]
    exe = tmp_path / "ax_manifest_tool"
    subprocess.check_call(["/usr/bin/g++", "-std=c++20", "-O1", "-o", str(exe), os.path.join(ref, "tools", "ax_manifest_tool.cpp")])
    manifests = [os.path.join(ref, "manifests", "kernels_sm89.json"), os.path.join(ref, "manifests", "kernels_sm90.json"),
                 os.path.join(ROOT, "manifests", "kernels_sm100.json")]
    many = []
    for m in manifests:
        many += ["--manifest", m]
    # the registry index the validation reads is generated from the same three manifests first (the reference's check.sh order)
    index = tmp_path / "graph_registry_index.json"
    out = subprocess.run([str(exe), "gen-registry-index", "--json-out", str(index), "--header-out", str(tmp_path / "graph_registry_index.hpp")] + many,
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    out = subprocess.run([str(exe), "validate-manifest", "--registry", str(index)] + many, capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
