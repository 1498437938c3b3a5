"""CPU-side checks of the drop-in boundary: the library loads without a GPU and exports every
symbol that include/asca_b200.h declares. No compute call is made here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "asca_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(asca_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_entry_points():
    names = declared_symbols()
    for n in ("asca_matmul", "asca_rmsnorm_fwd", "asca_rmsnorm_bwd", "asca_delta_fwd", "asca_delta_bwd",
              "asca_delta_step", "asca_moe_dispatch", "asca_moe_fwd", "asca_moe_bwd", "asca_gather_rows",
              "asca_scatter_rows", "asca_adamw", "asca_delta_scan_host", "asca_delta_bwd_dev_host",
              "asca_moe_forward_dev_host", "asca_moe_bwd_dev_host"):
        assert n in names


def test_library_loads_and_exports_every_declared_symbol():
    import asca_b200

    lib = asca_b200.load()
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    assert b"sm_100a" in lib.asca_version()


def test_no_gpu_means_a_loud_failure_not_a_fallback():
    import torch

    import asca_b200

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(asca_b200.AscaError):
        asca_b200.Gpu(0)


def test_null_context_is_rejected():
    import asca_b200

    lib = asca_b200.load()
    assert lib.asca_ctx_sync(ctypes.c_void_p(0)) == -1
    assert lib.asca_delta_ckpt_floats(8, 4096, 16, 128, 64) == 8 * 16 * 64 * 128 * 128
    assert lib.asca_delta_ckpt_floats(2, 70, 1, 16, 32) == 2 * 3 * 256


def test_product_never_imports_the_oracle():
    for p in (ROOT / "asca_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".h") and p.is_file():
            assert "oracle" not in p.read_text(), p
