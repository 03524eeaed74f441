"""The C-ABI library builds, loads and exports what ``include/gdn2_b200.h`` declares; argument
validation is exercised with calls that return before any device work (no GPU needed)."""

from __future__ import annotations

import ctypes
import pathlib
import re

import pytest

from gdn2_tilelang_b200 import _cabi

ROOT = pathlib.Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "gdn2_b200.h").read_text()


@pytest.fixture(scope="module")
def lib():
    return _cabi.load_library()


def declared_symbols():
    return sorted(set(re.findall(r"^(?:int|size_t|const char\*)\s+(gdn2_[a-z0-9_]+)\s*\(", HEADER, re.M)))


def test_header_and_binding_table_agree():
    assert declared_symbols() == sorted(_cabi.SIGNATURES)


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_is_exported(lib, name):
    assert getattr(lib, name) is not None


def test_abi_version_matches_header(lib):
    want = int(re.search(r"#define GDN2_B200_ABI_VERSION (\d+)", HEADER).group(1))
    assert lib.gdn2_abi_version() == want


def test_status_strings(lib):
    seen = {lib.gdn2_status_string(s) for s in range(0, -10, -1)}
    assert len(seen) == 10 and all(seen)
    assert lib.gdn2_status_string(-99) == b"unknown status"


def test_workspace_query(lib):
    f = lib.gdn2_prefill_workspace_bytes
    big = f(4, 16000, 16, 16, 128, 128, _cabi.GDN2_BF16, _cabi.PATH_TCGEN05_SERIAL)   # without the cut scan's segment records
    # per chunk-head: WQ 32 KiB + AQK 8 KiB + KG^T 16 KiB + U^T 16 KiB (fp16) + gamma_last 512 B (+ flag and list entry)
    per = 32768 + 8192 + 16384 + 16384 + 512 + 8
    nch = 4 * 16 * 250
    assert per * nch <= big <= per * nch + 8 * 1024
    assert f(1, 100, 1, 1, 128, 128, _cabi.GDN2_BF16, 0) == 0          # S not a multiple of 64
    assert f(1, 64, 1, 1, 36, 32, _cabi.GDN2_F32, 0) == 0              # DK not a multiple of 8
    assert f(1, 64, 1, 1, 256, 32, _cabi.GDN2_F32, 0) == 0             # DK too large for the chunkwise kernels
    assert f(1, 64, 1, 1, 64, 64, _cabi.GDN2_BF16, _cabi.PATH_TCGEN05) == 0   # tcgen05 family is D=128 only
    assert f(1, 64, 1, 1, 64, 64, _cabi.GDN2_BF16, _cabi.PATH_SIMT) > 0
    assert f(1, 64, 1, 1, 32, 24, 7, 0) == 0                           # bad dtype


def test_argument_validation_returns_status_without_device_work(lib):
    null = None
    one = ctypes.c_void_p(16)   # never dereferenced: validation fails first
    assert lib.gdn2_decode(null, one, one, one, one, one, one, one, 1, 1, 1, 1, 32, 32, 1, 1, 1.0, 0, None) == -1
    assert lib.gdn2_decode(one, one, one, one, one, one, one, one, 1, 1, 1, 1, 32, 32, 1, 1, 1.0, 9, None) == -3
    assert lib.gdn2_decode(one, one, one, one, one, one, one, one, 0, 1, 1, 1, 32, 32, 1, 1, 1.0, 0, None) == -2
    assert lib.gdn2_decode(one, one, one, one, one, one, one, one, 1, 1, 1, 1, 512, 32, 1, 1, 1.0, 0, None) == -2
    assert lib.gdn2_decode(one, one, one, one, one, one, one, one, 1, 4, 1, 1, 32, 32, 2, 4, 1.0, 0, None) == -2
    misaligned = ctypes.c_void_p(24)
    assert lib.gdn2_decode(one, one, one, one, one, one, misaligned, one, 1, 1, 1, 1, 128, 128, 1, 1, 1.0, 0, None) == -4
    assert lib.gdn2_chunk_prep(one, one, one, one, one, one, null, 0, 1, 64, 1, 1, 32, 32, 64, 1.0, 0, 0, None) == -1
    assert lib.gdn2_chunk_prep(one, one, one, one, one, one, one, 0, 1, 65, 1, 1, 32, 32, 65, 1.0, 0, 0, None) == -2
    assert lib.gdn2_chunk_prep(one, one, one, one, one, one, one, 0, 1, 64, 1, 1, 32, 32, 64, 1.0, 0, 2, None) == -8
    assert lib.gdn2_chunk_prep(one, one, one, one, one, one, misaligned, 1 << 30, 1, 64, 1, 1, 32, 32, 64, 1.0, 0, 0, None) == -4
    assert lib.gdn2_chunk_prep(one, one, one, one, one, one, one, 16, 1, 64, 1, 1, 32, 32, 64, 1.0, 0, 0, None) == -5
    assert lib.gdn2_prefill_scan(one, 16, null, one, null, null, 1, 64, 1, 1, 32, 32, 64, 0, 0, None) == -5
    assert lib.gdn2_prefill_scan(one, 1 << 30, null, null, null, null, 1, 64, 1, 1, 32, 32, 64, 0, 0, None) == -1
    assert lib.gdn2_chunk_output(one, 1 << 30, null, one, 1, 64, 1, 1, 32, 32, 64, 0, 0, None) == -1
    assert lib.gdn2_selftest_mma(null, one, one, None) == -1


def test_dtype_codes():
    import torch

    assert _cabi.dtype_code(torch.float32) == 0 and _cabi.dtype_code(torch.bfloat16) == 1
    with pytest.raises(TypeError):
        _cabi.dtype_code(torch.float64)


def test_batch_times_heads_limit_is_a_clear_status(lib):
    """The chunk-local kernels put (batch, head) on gridDim.y: more than 65535 pairs is refused as a bad shape
    before anything is enqueued, not reported as a failed launch."""
    one = ctypes.c_void_p(16)
    assert lib.gdn2_prefill_workspace_bytes(4095, 64, 16, 16, 128, 128, _cabi.GDN2_BF16, 0) > 0       # 65520 pairs
    assert lib.gdn2_prefill_workspace_bytes(4096, 64, 16, 16, 128, 128, _cabi.GDN2_BF16, 0) == 0      # 65536 pairs
    assert lib.gdn2_chunk_prep(one, one, one, one, one, one, one, 1 << 40, 4097, 64, 16, 16, 128, 128, 64, 1.0, 1, 0, None) == -2
    assert lib.gdn2_prefill_scan(one, 1 << 40, None, one, None, None, 4097, 64, 16, 16, 128, 128, 64, 1, 0, None) == -2
    # the one-call prefill: null pointers, head counts and strides are checked before anything is launched
    assert lib.gdn2_prefill_ragged(one, one, one, one, one, one, None, None, one, one, 1 << 40, 1, 100, 2, 2, 128, 128,
                                   100, 100, 1.0, 1, 0, None, None) == -1
    assert lib.gdn2_prefill_ragged(one, one, one, one, one, one, None, one, one, one, 1 << 40, 1, 100, 3, 2, 128, 128,
                                   100, 100, 1.0, 1, 0, None, None) == -2
    assert lib.gdn2_prefill_ragged(one, one, one, one, one, one, None, one, one, one, 1 << 40, 1, 100, 2, 2, 128, 128,
                                   99, 100, 1.0, 1, 0, None, None) == -2
    assert lib.gdn2_prefill_ragged(one, one, one, one, one, one, None, one, one, None, 0, 1, 100, 2, 2, 128, 128,
                                   100, 100, 1.0, 1, 0, None, None) == -1          # 64 whole tokens need a workspace
    # the scan in two parts takes part 1 or 2 only, and the same shape checks
    assert lib.gdn2_prefill_scan_part(one, 1 << 40, None, one, None, 1, 64, 16, 16, 128, 128, 64, 1, 0, 0, None) == -2
    assert lib.gdn2_prefill_scan_part(one, 1 << 40, None, one, None, 1, 64, 16, 16, 128, 128, 64, 1, 0, 3, None) == -2
    assert lib.gdn2_prefill_scan_part(one, 1 << 40, None, one, None, 4097, 64, 16, 16, 128, 128, 64, 1, 0, 1, None) == -2


def test_scan_segments_rule(lib):
    """How the tensor-core scan cuts a sequence: only with few (batch, head) pairs and long sequences, never for
    the SIMT family or the explicitly serial path; the workspace grows by the segment records and nothing else."""
    f = lib.gdn2_prefill_scan_segments
    bf = _cabi.GDN2_BF16
    assert f(4, 16000, 16, 128, 128, bf, _cabi.PATH_AUTO) == 2       # 64 pairs: 128 local blocks fit, the cut is guarded
    assert f(4, 16000, 8, 128, 128, bf, _cabi.PATH_AUTO) == 4        # 32 pairs: guarded as well
    assert f(5, 16000, 16, 128, 128, bf, _cabi.PATH_AUTO) == 1       # 80 pairs: two local blocks each would not fit
    assert f(4, 16000, 4, 128, 128, bf, _cabi.PATH_AUTO) == 5        # 16 pairs: 9 blocks each = 144, everything resident
    assert f(4, 16000, 2, 128, 128, bf, _cabi.PATH_AUTO) == 9        # 8 pairs: 17 blocks each = 136
    assert f(1, 16000, 1, 128, 128, bf, _cabi.PATH_AUTO) == 16       # capped
    assert f(2, 4096, 16, 128, 128, bf, _cabi.PATH_AUTO) == 2        # 32 pairs, 64 chunks: too short for a guarded cut in 4
    assert f(4, 64 * 15, 2, 128, 128, bf, _cabi.PATH_AUTO) == 1      # shorter than two 8-chunk segments
    assert f(4, 64 * 24, 2, 128, 128, bf, _cabi.PATH_AUTO) == 3
    assert f(4, 16000, 2, 128, 128, bf, _cabi.PATH_TCGEN05_SERIAL) == 1
    assert f(4, 16000, 2, 64, 64, bf, _cabi.PATH_AUTO) == 1          # SIMT family
    assert f(4, 100, 2, 128, 128, bf, _cabi.PATH_AUTO) == 0          # invalid shape
    n = lib.gdn2_prefill_scan_launches                                # what the scan launches for those cuts
    assert n(4, 16000, 16, 128, 128, bf, _cabi.PATH_AUTO) == 4       # guarded: decay check, first pass, chaining, redo
    assert n(4, 16000, 8, 128, 128, bf, _cabi.PATH_AUTO) == 4
    assert n(4, 16000, 2, 128, 128, bf, _cabi.PATH_AUTO) == 3        # every block resident: no guard
    assert n(4, 16000, 4, 128, 128, bf, _cabi.PATH_AUTO) == 3        # unguarded
    assert n(5, 16000, 16, 128, 128, bf, _cabi.PATH_AUTO) == 1
    assert n(4, 16000, 2, 64, 64, bf, _cabi.PATH_AUTO) == 1
    assert n(4, 100, 2, 128, 128, bf, _cabi.PATH_AUTO) == 0
    w = lib.gdn2_prefill_workspace_bytes
    cut, serial = w(4, 16000, 2, 2, 128, 128, bf, _cabi.PATH_TCGEN05), w(4, 16000, 2, 2, 128, 128, bf, _cabi.PATH_TCGEN05_SERIAL)
    want = 8 * 9 * (3 * 128 * 128 * 4 + 4)
    assert want <= cut - serial <= want + 1024
    out = (ctypes.c_int64 * 8)()
    assert lib.gdn2_prefill_workspace_layout(4, 16000, 2, 2, 128, 128, bf, _cabi.PATH_TCGEN05, out) == 0
    offs = list(out)
    assert offs == sorted(offs) and offs[0] == 0 and offs[7] == cut and offs[6] == serial
    assert lib.gdn2_prefill_workspace_layout(4, 100, 2, 2, 128, 128, bf, 0, out) == -2
    assert lib.gdn2_prefill_workspace_layout(4, 128, 2, 2, 128, 128, bf, 0, None) == -1


def test_wait_selftest_rejects_unbounded_limits(lib):
    assert lib.gdn2_selftest_wait(0, None, None) == -2
    assert lib.gdn2_selftest_wait(3_000_000_000, None, None) == -2
