"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

from speedup_thingy_b200 import _abi
from speedup_thingy_b200.build import build

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "rte_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rte_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_loads_and_exports_every_declared_symbol():
    lib_path = build()
    lib = ctypes.CDLL(str(lib_path))
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/rte_b200.h but not exported"
    assert sorted(_abi.PROTOTYPES) == declared, "ctypes prototypes and header declarations differ"


def test_argument_errors_do_not_need_a_gpu():
    lib = _abi.load()
    assert lib.rte_backend_name() == b"cuda_sm100a_ext"
    assert lib.rte_status_string(-1) == b"bad argument"
    # null pointers are rejected before any CUDA call
    assert lib.rte_cast_f32_bf16(None, None, 0, None) == -1
    args = _abi.GemmArgs()
    assert lib.rte_gemm_bf16(ctypes.byref(args), None) == -1


def test_product_path_fails_loudly_without_cuda():
    import pytest
    import torch
    from speedup_thingy_b200.config import ExperimentConfig
    from speedup_thingy_b200.engine import TrainEngine

    if torch.cuda.is_available():
        pytest.skip("needs a machine without CUDA")
    with pytest.raises(RuntimeError, match="CUDA is required"):
        TrainEngine(ExperimentConfig())
