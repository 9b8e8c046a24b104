"""The allocation-free decode entry point against the ordinary one, through the C ABI.

``cllo_gqa_decode_bf16_noalloc`` serves hosts that cannot hand the library a workspace (all device memory
already owned by a KV-cache pool, or a decode loop that must not trigger the synchronisation an allocation
implies): its split-KV partials live in a fixed ``__device__`` array inside the library.  The array is shared
by all calls and keeps its old contents, so the test calls twice in a row -- the second call runs over the
first call's leftovers -- and, collected last, also runs after every other test has used the device.
"""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import to_bits, to_dev

pytestmark = pytest.mark.gpu
SCALE = 1.0 / np.sqrt(128.0)


def _both(lib, q, k, v, B, S, Hq, Hkv, layout):
    from cuda_llm_ops_b200 import flash_gqa
    qd, kd, vd = to_dev(q), to_dev(k), to_dev(v)
    want = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
    got = torch.zeros((B, Hq, 128), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(flash_gqa.decode_workspace_bytes(B, S, Hq, Hkv), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    rc = lib.cllo_gqa_decode_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, want.data_ptr(), ws.data_ptr(),
                                  ws.numel(), B, S, Hq, Hkv, 128, layout, 0, None, None)
    assert rc == 0
    rc = lib.cllo_gqa_decode_bf16_noalloc(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), SCALE, got.data_ptr(),
                                          B, S, Hq, Hkv, 128, layout, 0, None)
    assert rc == 0
    torch.cuda.synchronize()
    return to_bits(got), to_bits(want)


def test_noalloc_entry_point_matches_the_workspace_entry_point_twice_in_a_row():
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    # two different problems back to back: the second one finds the first one's partials in the scratch
    for seed, (B, S, Hq, Hkv, layout) in enumerate([(3, 2000, 32, 4, 0), (2, 777, 16, 2, 1)]):
        q = ol.randn_bf16((B, Hq, 128), 900 + seed)
        shape = (B, S, Hkv, 128) if layout == 0 else (B, Hkv, S, 128)
        k, v = ol.randn_bf16(shape, 910 + seed), ol.randn_bf16(shape, 920 + seed)
        got, want = _both(lib, q, k, v, B, S, Hq, Hkv, layout)
        ol.assert_parity(got, want, "noalloc vs workspace entry point, call %d" % seed)
        ol.assert_parity(got, ol.decode(q, k, v, SCALE, layout), "noalloc vs oracle, call %d" % seed)


def test_noalloc_entry_point_refuses_more_workers_than_its_scratch_holds():
    from cuda_llm_ops_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(256, dtype=torch.bfloat16, device="cuda")
    rc = lib.cllo_gqa_decode_bf16_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), SCALE, x.data_ptr(),
                                          1, 1, 1, 1, 128, 0, 161, None)
    assert rc == _lib.E_WORKSPACE
    assert "workspace" in lib.cllo_status_string(rc).decode()
