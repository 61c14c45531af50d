"""The C-ABI library loads and exports every symbol include/pk100.h declares
(no compute calls here: this runs without a GPU)."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "pk100.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|long long|void|const char\s*\*)\s*(pk100_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "pk100_gemm" in names and "pk100_layer_norm" in names and len(names) >= 10


def test_library_exports_every_declared_symbol(pk):
    for name in declared_symbols():
        assert hasattr(pk.lib.lib, name), f"libpk100.so does not export {name}"


def test_binding_table_matches_header(pk):
    void_setters = ["pk100_set_gemm_cta_pairs", "pk100_set_gemm_cta_cap", "pk100_set_dependent_launch", "pk100_tensor_map_cache_stats"]
    assert sorted(list(pk.lib.SIGNATURES) + void_setters) == declared_symbols()


def test_argument_errors_need_no_gpu(pk):
    L = pk.lib
    # null pointers / bad shapes are rejected on the host before any launch
    assert L.lib.pk100_layer_norm(None, None, None, None, None, None, 0, 0.0, 8, 8, 8, None, 1e-5) == L.ERR_NULL
    assert L.lib.pk100_quantize_fp8_fixed(None, None, None, 16, 1.0) == L.ERR_NULL
    args = L.GemmArgs()
    assert L.lib.pk100_gemm(None, args) == L.ERR_NULL
