"""Parity against the reference's OWN device code: its CUDA runtime (engine/csrc/megakernel/qwen_runtime.cu), compiled
unchanged for sm_100a into oracle/_ref by `make -C oracle ref`, runs beside this library on the same inputs.
  * its matvec kernel with one-hot activations returns single dequantised weights (sums of one exact product and zeros
    are exact), which must equal this library's dequantiser bit for bit;
  * its matvec outputs on N(0,1) activations must agree with this library's within the 1e-5 relative L2 bound."""
from __future__ import annotations

import numpy as np
import pytest

from tests import oracle_libs
from vinf_3080ti_b200.gguf_types import CUDA_MATVEC_TYPES, GGUFTensorType as T
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu
ALL_TYPES = sorted(CUDA_MATVEC_TYPES, key=int)


@pytest.fixture(scope="module")
def ref_rt(codebooks):
    mod = oracle_libs.load_reference_cuda_module()
    if mod is None:
        pytest.skip("oracle/_ref/_cuda_qwen_runtime.so has not been built (make -C oracle ref REFERENCE=...)")
    return mod.Runtime(codebooks["iq3s_grid"])


@pytest.fixture(scope="module")
def rt(codebooks):
    from vinf_3080ti_b200.runtime import Runtime

    r = Runtime(codebooks["iq3s_grid"], codebooks)
    yield r
    r.close()


def _reference_qmv(ref_rt, raw, t, rows, cols, x):
    ntok = x.shape[0]
    ref_rt.upload("w", np.ascontiguousarray(raw).tobytes(), int(t), cols, rows)
    ref_rt.alloc("x", ntok * cols)
    ref_rt.alloc("y", ntok * rows)
    ref_rt.write("x", np.ascontiguousarray(x, dtype=np.float32).tobytes())
    ref_rt.qmv("w", "x", "y", ntok)
    ref_rt.synchronize()
    return np.frombuffer(ref_rt.read("y"), dtype=np.float32).reshape(ntok, rows).copy()


@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_dequantised_values_equal_the_reference_device_dequantiser(rt, ref_rt, t):
    rng = np.random.default_rng(900 + int(t))
    rows, cols = 37, 512
    raw = synthetic_blocks(t, rows, cols, rng)
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("deq", rows * cols)
    rt.dequantize("w", "deq")
    rt.synchronize()
    mine = rt.read_array("deq").reshape(rows, cols)
    picked = rng.choice(cols, size=64, replace=False)
    for start in range(0, 64, 8):
        x = np.zeros((8, cols), dtype=np.float32)
        x[np.arange(8), picked[start : start + 8]] = 1.0
        theirs = _reference_qmv(ref_rt, raw, t, rows, cols, x)  # [8][rows]: column picked[start + k] of W
        want = np.ascontiguousarray(mine[:, picked[start : start + 8]].T)
        # (a sum cannot return -0.0: adding +0.0 on both sides takes the sign of zero out of the comparison)
        assert np.array_equal((theirs + np.float32(0.0)).view(np.uint32), (want + np.float32(0.0)).view(np.uint32))


@pytest.mark.parametrize("t,rows,cols,ntok", [(t, 129, 1024, m) for t in ALL_TYPES for m in (1, 4)] +
                         [(T.Q4_K, 17408, 5120, 1), (T.Q3_K, 17408, 5120, 4), (T.Q6_K, 6144, 5120, 8), (T.IQ4_XS, 2048, 5120, 8)],
                         ids=lambda v: getattr(v, "name", str(v)))
def test_matvec_agrees_with_the_reference_kernel(rt, ref_rt, t, rows, cols, ntok):
    rng = np.random.default_rng(rows + int(t) + ntok)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    theirs = _reference_qmv(ref_rt, raw, t, rows, cols, x).astype(np.float64)
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", x)
    rt.qmv("w", "x", "y", ntok)
    rt.synchronize()
    mine = rt.read_array("y").reshape(ntok, rows).astype(np.float64)
    assert float(np.linalg.norm(mine - theirs) / np.linalg.norm(theirs)) <= 1e-5
