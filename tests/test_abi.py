"""The C-ABI library loads, exports every declared symbol and validates before launching.

No compute call happens here: every b200fa_fwd / b200fa_bwd invocation below is rejected by
argument validation, which the library performs before it touches CUDA."""

import ctypes
import os
import re

import pytest

from torch_mojo_backend_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200fa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200fa_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert _lib.version() == 2
    assert _lib.launch_count() == 0 or _lib.launch_count() > 0


def test_strerror_covers_all_codes():
    seen = set()
    for code in range(0, -10, -1):
        msg = _lib.strerror(code)
        assert msg and "unknown" not in msg
        seen.add(msg)
    assert len(seen) == 10
    assert "unknown" in _lib.strerror(-99)


def test_workspace_formula():
    # 2 x (B*Hq*Spad) fp32 row statistics, Spad = ceil(S/128)*128 (the reference's scratch,
    # aten_fast.py:7314-7324, minus its fp32 dQ accumulator: dQ accumulates in tensor memory)
    B, Hq, Hkv, S, D = 8, 12, 12, 1024, 64
    rows = B * Hq * 1024
    assert _lib.bwd_workspace_bytes(B, Hq, Hkv, S, D, _lib.BF16) == 2 * rows * 4
    assert _lib.bwd_workspace_bytes(1, 1, 1, 65, 64, _lib.BF16) == 2 * 512
    assert _lib.bwd_workspace_bytes(0, 1, 1, 65, 64, _lib.BF16) == 0


def _t4(ptr, shape, stride=None):
    if stride is None:
        stride = (shape[1] * shape[2] * shape[3], shape[2] * shape[3], shape[3], 1)
    return _lib.Tensor4.make(ptr, shape, stride)


FAKE = 0x7F0000000000  # never dereferenced: validation rejects the call first


@pytest.mark.parametrize(
    "mutate,expected",
    [
        (dict(dtype=7), _lib.ERR_BAD_DTYPE),
        (dict(q_shape=(1, 2, 128, 96)), _lib.ERR_UNSUPPORTED),  # head_dim not 64/128
        (dict(k_shape=(1, 3, 128, 64), q_shape=(1, 4, 128, 64)), _lib.ERR_BAD_SHAPE),  # Hq % Hkv
        (dict(causal=3), _lib.ERR_UNSUPPORTED),  # not one of B200FA_CAUSAL_*
        (dict(q_stride=(0, 8192, 64, 1), q_shape=(2, 2, 128, 64), k_shape=(2, 2, 128, 64)), _lib.ERR_BAD_STRIDE),  # broadcast batch
        (dict(k_stride=(16384, 0, 64, 1)), _lib.ERR_BAD_STRIDE),  # broadcast heads
        (dict(out_stride=(16384, 64, 64, 1)), _lib.ERR_BAD_STRIDE),  # output heads overlap one another
        (dict(dropout=(1.0, 1, 0)), _lib.ERR_UNSUPPORTED),
        (dict(dropout=(-0.5, 1, 0)), _lib.ERR_UNSUPPORTED),
        (dict(q_shape=(65535, 65535, 128, 64), k_shape=(65535, 65535, 128, 64)), _lib.ERR_BAD_SHAPE),  # grid index overflow
        (dict(scale=0.0), _lib.ERR_UNSUPPORTED),
        (dict(scale=float("nan")), _lib.ERR_UNSUPPORTED),
        (dict(q_stride=(16384, 8192, 64, 2)), _lib.ERR_BAD_STRIDE),  # head_dim stride must be 1
        (dict(q_stride=(16388, 8196, 68, 1)), _lib.ERR_BAD_STRIDE),  # rows not 16-byte multiples
        (dict(q_ptr=FAKE + 2), _lib.ERR_MISALIGNED),
        (dict(q_ptr=0), _lib.ERR_NULL),
        (dict(lse=0), _lib.ERR_NULL),
        (dict(v_shape=(1, 2, 128, 128)), _lib.ERR_BAD_SHAPE),
    ],
)
def test_forward_validates_before_launch(mutate, expected):
    q_shape = mutate.get("q_shape", (1, 2, 128, 64))
    k_shape = mutate.get("k_shape", (1, 2, 128, 64))
    v_shape = mutate.get("v_shape", k_shape)
    q = _t4(mutate.get("q_ptr", FAKE), q_shape, mutate.get("q_stride"))
    k = _t4(FAKE + 0x100000, k_shape, mutate.get("k_stride"))
    v = _t4(FAKE + 0x200000, v_shape)
    out = _t4(FAKE + 0x300000, q_shape, mutate.get("out_stride"))
    before = _lib.launch_count()
    rc = _lib.fwd(q, k, v, out, mutate.get("lse", FAKE + 0x400000), mutate.get("dtype", _lib.BF16),
                  mutate.get("causal", True), mutate.get("scale", 0.125), 0, 0, dropout=mutate.get("dropout"))
    assert rc == expected, _lib.strerror(rc)
    assert _lib.launch_count() == before


def test_backward_rejects_small_or_missing_workspace():
    shape = (1, 2, 128, 64)
    t = [_t4(FAKE + i * 0x100000, shape) for i in range(8)]
    need = _lib.bwd_workspace_bytes(1, 2, 2, 128, 64, _lib.BF16)
    for ws_ptr, ws_bytes in ((0, need), (FAKE + 0x900000, need - 1), (FAKE + 0x900010, need)):
        rc = _lib.bwd(t[0], t[1], t[2], t[3], t[4], FAKE + 0xA00000, t[5], t[6], t[7], ws_ptr, ws_bytes, _lib.BF16,
                      True, 0.125, 0, 0)
        assert rc == _lib.ERR_WORKSPACE


def test_split_kv_entry_point_validates_before_launch():
    q = _t4(FAKE, (1, 8, 1, 128))
    k = _t4(FAKE + 0x100000, (1, 2, 4096, 128))
    out = _t4(FAKE + 0x300000, (1, 8, 1, 128))
    need = _lib.fwd_splitkv_workspace_bytes(1, 8, 2, 1, 4096, 128)
    assert need > 0 and need % 256 == 0
    before = _lib.launch_count()
    assert _lib.fwd_splitkv(q, k, k, out, FAKE + 0x400000, 0, need, _lib.BF16, False, 0.1, 0, 0) == _lib.ERR_WORKSPACE
    assert _lib.fwd_splitkv(q, k, k, out, FAKE + 0x400000, FAKE + 0x500000, need - 1, _lib.BF16, False, 0.1, 0,
                            0) == _lib.ERR_WORKSPACE
    # 8 query rows x 4 heads per kv head = 32 rows: more than one split-KV thread block carries
    q32 = _t4(FAKE, (1, 8, 8, 128))
    assert _lib.fwd_splitkv(q32, k, k, _t4(FAKE + 0x300000, (1, 8, 8, 128)), FAKE + 0x400000, FAKE + 0x500000,
                            1 << 30, _lib.BF16, False, 0.1, 0, 0) == _lib.ERR_UNSUPPORTED
    assert _lib.launch_count() == before


def _splits_of(B, Hq, Hkv, Sq, Sk, D):
    """The split count the library chose, read back from the workspace size: fp32 partial outputs
    and (max, sum) pairs per (row, split), one counter per (batch, KV head), each 256-byte aligned."""
    total = _lib.fwd_splitkv_workspace_bytes(B, Hq, Hkv, Sq, Sk, D)
    al = lambda x: (x + 255) // 256 * 256
    rows = B * Hq * Sq
    for n in range(1, 65):
        if al(rows * n * D * 4) + al(rows * n * 8) + al(B * Hkv * 4) == total:
            return n
    raise AssertionError(f"workspace of {total} bytes fits no split count")


def test_split_count_fills_whole_waves_of_the_grid():
    # few (batch, KV head) pairs over a long cache: one wave of 3 x 148 thread blocks, not one and a bit
    n = _splits_of(1, 32, 8, 1, 131072, 128)
    assert 8 * n <= 444 < 8 * (n + 8) and 131072 // n >= 256
    # many pairs: a handful of long splits (the fixed cost per thread block outweighs a fuller last wave)
    assert _splits_of(64, 32, 8, 1, 8192, 128) <= 8
    # more than eight rows per KV head: two thread blocks per SM
    n16 = _splits_of(1, 32, 2, 1, 131072, 128)
    assert 2 * n16 <= 296
    # a split is never shorter than 256 keys (but for the last one)
    assert _splits_of(1, 8, 8, 1, 600, 64) <= 3 and _splits_of(2, 4, 4, 1, 200, 64) == 1


def test_forward_kernel_shape_setter():
    assert _lib.fwd_tiles() in (0, 1, 2)
    for tiles in (1, 2, 0):
        _lib.set_fwd_tiles(tiles)
        assert _lib.fwd_tiles() == tiles
    _lib.set_fwd_tiles(7)   # anything else means "chosen per problem"
    assert _lib.fwd_tiles() == 0


def test_wait_budget_and_status_helpers():
    default = _lib.wait_budget()
    assert default > 0
    _lib.set_wait_budget(12345)
    assert _lib.wait_budget() == 12345
    _lib.set_wait_budget(0)   # back to the default (or B200FA_WAIT_BUDGET)
    assert _lib.wait_budget() == default
    assert _lib.status_to_error(0) == _lib.OK
    assert _lib.status_to_error(0x57410100) == _lib.ERR_TIMEOUT
    assert _lib.status_to_error(0x414C0000) == _lib.ERR_CUDA
    # the self-test kernel is refused without a status word or with a silly budget, before any launch
    before = _lib.launch_count()
    assert _lib.selftest_wait_timeout(0, 1000, 0, 0) == _lib.ERR_NULL
    assert _lib.selftest_wait_timeout(FAKE, 0, 0, 0) == _lib.ERR_UNSUPPORTED
    assert _lib.launch_count() == before


def test_dropout_threshold_quantises_to_256ths():
    assert [_lib.dropout_threshold(p) for p in (0.0, 0.001, 0.1, 0.25, 0.5, 0.999)] == [0, 0, 26, 64, 128, 255]


def test_valid_call_without_gpu_reports_cuda_error_not_success():
    """With valid arguments and no device the library must fail loudly (never pretend)."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present; this checks the no-GPU failure mode")
    shape = (1, 2, 128, 64)
    t = [_t4(FAKE + i * 0x100000, shape) for i in range(4)]
    rc = _lib.fwd(t[0], t[1], t[2], t[3], FAKE + 0x800000, _lib.BF16, True, 0.125, 0, 0)
    assert rc in (_lib.ERR_CUDA, _lib.ERR_UNSUPPORTED)


def test_struct_layout_matches_header():
    assert ctypes.sizeof(_lib.Tensor4) == 8 + 32 + 32
    assert _lib.Tensor4.shape.offset == 8 and _lib.Tensor4.stride.offset == 40
