"""libq35b.so loads without a GPU and exports every function include/q35b_nvfp4.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "q35b_nvfp4.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"Q35B_API\s+[\w\s\*]+?\b(q35b_\w+)\s*\(", text)))


def test_header_lists_functions():
    names = declared_functions()
    assert "q35b_gemv_w4a16_bf16" in names and "q35b_gemm_w4a4_bf16" in names and len(names) >= 20


def test_every_symbol_exported(engine):
    L = engine.lib()
    missing = [n for n in declared_functions() if not hasattr(L, n)]
    assert not missing, missing
    assert b"q35b" in L.q35b_version()


def test_argument_errors_without_gpu(engine):
    L = engine.lib()
    h = ctypes.c_void_p()
    assert L.q35b_weight_create(None, None, 1.0, 1.0, 8, 16, 0, 1, ctypes.byref(h)) == 1
    assert b"null" in L.q35b_last_error()
    buf = (ctypes.c_uint8 * 64)()
    assert L.q35b_weight_create(buf, buf, 1.0, 1.0, 8, 24, 0, 1, ctypes.byref(h)) == 2  # cols % 16 != 0
    assert L.q35b_weight_create(buf, buf, 1.0, 1.0, 8, 16, 3, 2, ctypes.byref(h)) == 1  # bad shard
    assert L.q35b_gemv_w4a16_bf16(None, None, 1, None, -1, None) == 1


def test_shard_ranges(engine):
    for n in (2560, 3584, 18432, 9216, 32768, 100, 129):
        for g in (1, 2, 4, 8):
            spans = [engine.shard_range(n, i, g) for i in range(g)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (b0, c0), (b1, _) in zip(spans, spans[1:]):
                assert b0 + c0 == b1
            for b, c in spans[:-1]:
                assert b % 128 == 0
            counts = [c for _, c in spans]
            if n % 128 == 0:
                assert max(counts) - min(counts) <= 128


def test_no_cpu_fallback(engine):
    import torch

    if torch.cuda.is_available():
        return
    import numpy as np
    import pytest

    with pytest.raises(engine.Q35bError):
        engine.Nvfp4Weight.from_host(np.zeros((8, 8), np.uint8), np.zeros((8, 1), np.uint8), 1.0)
