"""The allocation-free LM-head entry point, vqm_qmv_argmax_static, against the regular vqm_qmv_argmax.

Some users of the library may not call the CUDA allocator where they run the LM head (a serving loop under a
no-allocation rule, a process that handed out all of its GPU memory at start-up, a plugin restricted to its
host's buffers).  For them the scratch the fused argmax needs is a fixed array inside the library.  This test
drives that entry point through the C ABI with caller-owned device pointers, twice in a row (the array keeps the
previous call's contents), and requires the same logits bit for bit and the same token ids as the regular path.
It lives in the last-collected file so that a run stopping at the first failure has already run everything else.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from vinf_3080ti_b200 import _capi
from vinf_3080ti_b200.gguf_types import GGUFTensorType as T
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_the_regular_fused_argmax_twice(codebooks):
    from vinf_3080ti_b200.runtime import Runtime

    lib = _capi.load()
    rt = Runtime(codebooks["iq3s_grid"], codebooks)
    rng = np.random.default_rng(2024)
    rows, cols = 6001, 2048
    raw = synthetic_blocks(T.Q6_K, rows, cols, rng)
    rt.upload("w", raw, int(T.Q6_K), cols, rows)
    w_addr = rt.tensor_info("w")[0]
    for name, n in (("x", 8 * cols), ("y_ref", 8 * rows), ("y_new", 8 * rows), ("ids", 8), ("vals", 8), ("status", 4)):
        rt.alloc(name, n)
    ptr = {name: rt.buffer_ptr(name)[0] for name in ("x", "y_new", "ids", "vals", "status")}
    for call, ntok in enumerate((4, 7)):  # two calls in a row, different widths, fresh activations
        x = synthetic_activations(ntok, cols, rng)
        rt.write("x", x)
        want_ids = rt.qmv_argmax("w", "x", "y_ref", ntok)
        want_vals = rt.argmax_fetch(ntok, with_values=True)[1]
        rt.zero("y_new")
        rc = lib.vqm_qmv_argmax_static(int(T.Q6_K), ctypes.c_void_p(w_addr), rows, cols, ctypes.c_void_p(ptr["x"]),
                                       ctypes.c_void_p(ptr["y_new"]), ntok, None, ctypes.c_void_p(ptr["ids"]),
                                       ctypes.c_void_p(ptr["vals"]), ctypes.c_void_p(ptr["status"]), ctypes.c_void_p(rt.stream()))
        _capi.check(rc)
        rt.synchronize()
        got_ids = np.frombuffer(rt.read("ids"), dtype=np.int32)[:ntok].tolist()
        got_vals = rt.read_array("vals")[:ntok].tolist()
        assert got_ids == want_ids, (call, got_ids, want_ids)
        assert got_vals == want_vals
        assert np.array_equal(rt.read_array("y_new", ntok * rows).view(np.uint32), rt.read_array("y_ref", ntok * rows).view(np.uint32))
        assert np.frombuffer(rt.read("status"), dtype=np.uint32)[0] == 0
    # the property the entry point exists for: a call (here the ids-only form, y = NULL) leaves the device's free memory as it was
    free_before = rt.mem_info()[0]
    rc = lib.vqm_qmv_argmax_static(int(T.Q6_K), ctypes.c_void_p(w_addr), rows, cols, ctypes.c_void_p(ptr["x"]), None, ntok, None,
                                   ctypes.c_void_p(ptr["ids"]), None, ctypes.c_void_p(ptr["status"]), ctypes.c_void_p(rt.stream()))
    _capi.check(rc)
    rt.synchronize()
    assert rt.mem_info()[0] == free_before
    assert np.frombuffer(rt.read("ids"), dtype=np.int32)[:ntok].tolist() == want_ids
    # sizes beyond the maximum are refused with a clear error, nothing is launched
    rc = lib.vqm_qmv_argmax_static(int(T.Q6_K), ctypes.c_void_p(w_addr), rows, cols, ctypes.c_void_p(ptr["x"]), None, 9, None,
                                   ctypes.c_void_p(ptr["ids"]), None, ctypes.c_void_p(ptr["status"]), ctypes.c_void_p(rt.stream()))
    assert rc == _capi.ERR_VALUE and b"ntok" in lib.vqm_last_error()
    rt.close()
