"""The C-ABI libraries load and export every symbol their headers declare (no compute: runs without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

from dphpc_b200 import capi

ROOT = Path(__file__).resolve().parent.parent


def declared(header: str, prefix: str):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(rf"\b({prefix}\w+)\s*\(", text)))


def test_engine_exports_every_declared_symbol():
    lib = capi.load_engine_lib()
    names = declared("sddmm_b200.h", "sddmm_b200_")
    assert len(names) >= 20
    assert sorted(capi.ENGINE_SYMBOLS) == names
    for n in names:
        assert hasattr(lib, n), n


def test_dataset_lib_exports_every_declared_symbol():
    lib = capi.load_dataset_lib()
    names = declared("sddmm_datasets.h", "sddmm_dataset_")
    assert sorted(capi.DATASET_SYMBOLS) == names
    for n in names:
        assert hasattr(lib, n), n


def test_plan_struct_matches_header_layout():
    # field order and widths of sddmm_b200_plan_info as declared in the header
    text = (ROOT / "include" / "sddmm_b200.h").read_text()
    body = re.search(r"typedef struct sddmm_b200_plan_info \{(.*?)\} sddmm_b200_plan_info;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for ty, names in re.findall(r"(int64_t|int32_t)\s+([^;]+);", body):
        for n in names.split(","):
            fields.append((n.strip().split("[")[0], ty))
    got = [(n, "int64_t" if (t is ctypes.c_int64 or getattr(t, "_type_", None) is ctypes.c_int64) else "int32_t")
           for n, t in capi.PlanInfo._fields_]
    assert got == fields


def test_no_cpu_fallback_without_device():
    if capi.device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(capi.SddmmError) as ei:
        capi.Engine(0, "fp32")
    assert ei.value.code == 4  # SDDMM_B200_ERR_CUDA: the product path fails loudly, it never computes on the CPU


def test_product_sources_do_not_reach_into_oracle():
    # the engine, the bindings and the C++ competitor never include/import/open anything under oracle/
    pat = re.compile(r"oracle[/_.]|liboracle|libsddmm_ref")
    for p in list((ROOT / "dphpc_b200").rglob("*")) + list((ROOT / "include").rglob("*")):
        if p.suffix in {".py", ".cu", ".cuh", ".cpp", ".hpp", ".h"}:
            assert not pat.search(p.read_text()), p
