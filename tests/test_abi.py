"""The C-ABI library loads and exports every symbol include/jgq.h declares.
Runs without a GPU: only host-side argument validation is exercised."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def jlib():
    from jax_gptq_b200 import build
    build.build()
    from jax_gptq_b200 import _lib
    return _lib


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'jgq.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(jgq_\w+)\s*\(', text)))


def test_header_symbols_exported(jlib):
    names = declared_symbols()
    assert len(names) >= 16
    raw = ctypes.CDLL(jlib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f'{n} declared in jgq.h but not exported'
    assert set(names) == set(jlib.SIGNATURES), 'ctypes signature table out of sync with jgq.h'
    assert jlib.lib.jgq_version() >= 100


def test_validation_errors_without_gpu(jlib):
    lib = jlib.lib
    # odd packed-axis length (the reference's shapes would not broadcast either)
    assert lib.jgq_pack_int4(1, jlib.U8, 1, 1, 3, 1, None) == -1
    assert b'odd' in lib.jgq_last_error()
    assert lib.jgq_pack_int4(1, jlib.F32, 1, 1, 4, 1, None) == -1
    # empty inputs are accepted and launch nothing
    assert lib.jgq_pack_int4(None, jlib.U8, None, 0, 4, 8, None) == 0
    assert lib.jgq_unpack_int4(None, None, 4, 0, 8, None) == 0
    # K not a multiple of block_size (gptq.py:132-133 slices fixed-size blocks)
    assert lib.jgq_gptq_quantize(1, 1, 1, 1, 100, 8, 16, 15, 1, jlib.F32, None, 1, 1 << 20, None) == -1
    assert lib.jgq_gptq_quantize(1, 1, 1, 1, 128, 8, 256, 15, 1, jlib.F32, None, 1, 1 << 20, None) == -1
    # odd contraction length for the matmul
    assert lib.jgq_w4_matmul(1, jlib.F16, 1, 1, 1, jlib.F16, 1, 1, 8, 7, 0, 1, 1 << 20, None) == -1
    assert lib.jgq_w4_matmul(1, jlib.U8, 1, 1, 1, jlib.F16, 1, 1, 8, 8, 0, 1, 1 << 20, None) == -1
    # workspace too small / size queries
    assert lib.jgq_damp_invert_workspace_bytes(768) >= 768 * 768 * 4
    assert lib.jgq_damp_invert(1, 8, 1, 768, 0.01, 1, 256, 16, 1, None) == -3
    assert lib.jgq_hessian_finalize(1, 16, 0.0, None) == -1
    # activation-order gathers: in-place calls and more rows than a grid dimension holds are refused, empty ones accepted
    assert lib.jgq_gather_rows(256, 8, 64, 512, 256, None) == -1
    assert lib.jgq_gather_rows(256, 70000, 64, 512, 1024, None) == -5
    assert lib.jgq_gather_rows(None, 0, 64, None, None, None) == 0
    assert lib.jgq_permute_sym(256, 16, 512, 256, None) == -1
    assert lib.jgq_permute_sym(256, 0, 512, 1024, None) == -1
    with pytest.raises(jlib.JgqError):
        jlib.check(-1)
