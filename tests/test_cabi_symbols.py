"""The C-ABI library loads without a GPU and exports exactly what include/*.h declares."""
import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names |= set(re.findall(r"\b(cllo_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("cllo_gqa_decode_bf16", "cllo_gqa_combine_bf16", "cllo_gqa_prefill_fwd_bf16",
                 "cllo_gqa_decode_workspace_bytes", "cllo_device_status"):
        assert must in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    for name in _declared():
        assert hasattr(lib, name), name


def test_python_binding_covers_every_declared_symbol(built_library):
    from cuda_llm_ops_b200 import _lib
    assert set(_declared()) <= set(_lib.declared_symbols())
    _lib.load()


def test_argument_validation_needs_no_gpu(built_library):
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    assert lib.cllo_version() >= 100
    assert lib.cllo_gqa_decode_bf16(None, None, None, 1.0, None, None, 0, 1, 1, 1, 1, 128, 0, 0, None, None) == _lib.E_BAD_ARG
    assert lib.cllo_gqa_combine_bf16(None, 1, None, 1, 128, None) == _lib.E_BAD_ARG
    assert lib.cllo_gqa_prefill_fwd_bf16(None, None, None, 1.0, 0, None, None, 1, 1, 1, 1, 1, 128, None) == _lib.E_BAD_ARG
    # a zero or non-finite softmax scale is refused by the forward launchers (masking multiplies infinities by it)
    for bad in (0.0, float("inf"), float("nan")):
        assert lib.cllo_gqa_prefill_fwd_bf16(1 << 20, 1 << 20, 1 << 20, bad, 1, 1 << 20, None, 1, 256, 256, 4, 4, 128,
                                             None) == _lib.E_BAD_ARG
        assert lib.cllo_mla_prefill_fwd_bf16(1 << 20, 1 << 20, 1 << 20, bad, 1, 1 << 20, None, 1, 256, 256, 4, 4, 192,
                                             128, None) == _lib.E_BAD_ARG
    assert lib.cllo_status_string(_lib.E_WORKSPACE).decode().startswith("workspace")
    # peer exchange: null tables, rank outside the world, epoch 0, too many peers
    two = (ctypes.c_void_p * 2)(1 << 20, 2 << 20)
    ex = lib.cllo_gqa_exchange_combine_bf16
    assert ex(None, None, None, 0, 2, 1, None, 1, 64, 8, 128, None) == _lib.E_BAD_ARG
    assert ex(1 << 20, two, two, 2, 2, 1, 1 << 20, 1, 64, 8, 128, None) == _lib.E_BAD_ARG
    assert ex(1 << 20, two, two, 0, 17, 1, 1 << 20, 1, 64, 8, 128, None) == _lib.E_BAD_ARG
    assert ex(1 << 20, two, two, 0, 2, 1, 1 << 20, 1, 64, 8, 64, None) == _lib.E_UNSUPPORTED
    assert ex(1 << 20, two, two, 0, 2, 1, 1 << 20, 1, 64, 6, 128, None) == _lib.E_BAD_ARG       # Hq % Hkv
    assert ex(1 << 20, two, two, 0, 2, 1, 1 << 20, 300, 8, 8, 128, None) == _lib.E_UNSUPPORTED  # too many units
    # the fused form validates the exchange tables before anything else
    fused = lib.cllo_gqa_decode_sharded_bf16
    assert fused(1 << 20, 1 << 20, 1 << 20, 1.0, 1 << 20, None, 0, 1, 64, 64, 8, 128, 0, 0, None, None, 0, 2, 1,
                 None) == _lib.E_BAD_ARG
    assert lib.cllo_gqa_shard_gather_bytes(8, 1, 64, 128) == 2 * 8 * 64 * 130 * 4
    assert lib.cllo_gqa_shard_flag_bytes(8) == (8 * 256 + 1) * 4
    assert lib.cllo_gqa_shard_flag_bytes(17) == 0
    assert lib.cllo_set_exchange_wait_limit(0) == 0


def test_decode_plan_balances_tiles(built_library):
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    plan = (ctypes.c_int * 6)()
    # the headline decode shape on a 148-SM part
    assert lib.cllo_gqa_decode_plan(60, 4096, 128, 8, 128, 0, 148, plan) == 0
    W, n_t, T, merge, tok = plan[0], plan[1], plan[2] | (plan[3] << 32), plan[4], plan[5]
    # 480 (batch, kv head) units: the library picks 120 blocks of four whole units each, nothing to merge
    assert (W, tok, n_t, T, merge) == (120, 64, 64, 60 * 8 * 64, 0)
    # an explicit count is taken as given; shares differ by at most one tile
    assert lib.cllo_gqa_decode_plan(60, 4096, 128, 8, 128, 148, 148, plan) == 0 and plan[0] == 148 and plan[4] == 1
    W = 148
    shares = [((w + 1) * T) // W - (w * T) // W for w in range(W)]
    assert max(shares) - min(shares) <= 1 and sum(shares) == T
    # one long sequence, 8 kv heads: 128 blocks, every head cut into 16 equal pieces
    assert lib.cllo_gqa_decode_plan(1, 1 << 20, 64, 8, 128, 0, 148, plan) == 0 and plan[0] == 128 and plan[4] == 1
    # fewer tiles than workers: the worker count shrinks to the tile count
    assert lib.cllo_gqa_decode_plan(1, 100, 4, 1, 128, 0, 148, plan) == 0 and plan[0] == 2
    # whole units per worker: no merge pass
    assert lib.cllo_gqa_decode_plan(4, 1024, 32, 8, 128, 32, 148, plan) == 0 and plan[4] == 0
    assert lib.cllo_gqa_decode_plan(1, 64, 6, 4, 128, 0, 148, plan) == _lib.E_BAD_ARG
    assert lib.cllo_gqa_decode_plan(1, 64, 4, 4, 64, 0, 148, plan) == _lib.E_UNSUPPORTED
    # 4 KB of arrival counters, then two partial slots per worker
    assert lib.cllo_gqa_decode_workspace_bytes(60, 4096, 128, 8, 128, 148) == 4096 + 148 * 2 * 16 * 130 * 4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from cuda_llm_ops_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
