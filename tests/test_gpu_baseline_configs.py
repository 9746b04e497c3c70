"""GPU parity on the benchmark's own configurations, every case against the CPU oracle (never against this library).

  * the fused matvec + argmax of the full-size LM head (Q6_K 151936 x 5120, four activation rows): token ids equal the
    argmax of the oracle's fp64 logits, logits within the 1e-5 relative L2 bar
    (engine/src/vinf/qwen_gpu.py:1080-1086 is the caller this stands for);
  * the matvec kernels' OWN dequantisation, read back through one-hot activations: a sum of one exact product and
    zeros is exact, so y[t][r] is the dequantised weight W[r][c_t] and must equal the oracle's value exactly - for
    every type, with one and with eight activation rows, on a short tensor and on a tall one (the launcher picks
    different row-group heights for them);
  * the mixed layer: all seven tensors at 1, 2, 4 and 8 activation rows;
  * the IQ sweep: all five tensors at 1 and 8 activation rows.
"""
from __future__ import annotations

import numpy as np
import pytest

from oracle import dequant_np as O
from tests import oracle_libs
from vinf_3080ti_b200.gguf_types import TRAITS, GGUFTensorType as T
from vinf_3080ti_b200.synth import IQ_SWEEP, LAYER_SET, LM_HEAD, synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu
REL_L2 = 1e-5
ALL_TYPES = sorted(TRAITS)


@pytest.fixture(scope="module")
def rt(codebooks):
    from vinf_3080ti_b200.runtime import Runtime

    runtime = Runtime(codebooks["iq3s_grid"], codebooks)
    yield runtime
    runtime.close()


@pytest.fixture(scope="module")
def clib():
    return oracle_libs.load_c_oracle()


def rel_l2(got: np.ndarray, ref: np.ndarray) -> float:
    return float(np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-300))


def _qmv(rt, raw, t, rows, cols, x):
    ntok = x.shape[0]
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", np.ascontiguousarray(x, dtype=np.float32))
    rt.qmv("w", "x", "y", ntok)
    rt.synchronize()
    return rt.read_array("y").reshape(ntok, rows).copy()


def test_full_size_lm_head_token_ids_equal_the_oracle(rt, clib, codebooks):
    _, t, rows, cols = LM_HEAD
    ntok = 4
    for seed in range(4):  # near-ties of the two largest logits are a property of the inputs, not of a kernel: reseed
        rng = np.random.default_rng(4000 + seed)
        raw = synthetic_blocks(t, rows, cols, rng)
        x = synthetic_activations(ntok, cols, rng)
        ref = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
        top2 = np.partition(ref, rows - 2, axis=1)[:, -2:]
        if np.all(top2[:, 1] - top2[:, 0] >= 1e-4 * np.abs(top2[:, 1])):
            break
    else:
        pytest.fail("four seeds in a row gave near-tied logits")
    want = [int(v) for v in oracle_libs.c_argmax_rows(clib, ref)]
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", x)
    assert rt.qmv_argmax("w", "x", "y", ntok) == want
    assert rel_l2(rt.read_array("y").reshape(ntok, rows), ref) <= REL_L2
    assert rt.qmv_argmax("w", "x", None, ntok) == want  # ids only, logits not stored
    rt.qmv("w", "x", "y", ntok)  # and the unfused pair of calls the reference makes
    assert rt.argmax_rows("y", rows, ntok) == want
    rt.free("w")


@pytest.mark.parametrize("rows", [70, 9600], ids=["short", "tall"])
@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_matvec_kernels_dequantise_exactly(rt, codebooks, t, rows):
    rng = np.random.default_rng(7000 + 31 * int(t) + rows)
    cols = 512
    raw = synthetic_blocks(t, rows, cols, rng)
    want = O.dequantize(raw, int(t), rows * cols, codebooks).astype(np.float32).reshape(rows, cols)
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("x", 8 * cols)
    rt.alloc("y", 8 * rows)
    order = rng.permutation(cols)
    # eight columns per launch, every column of the tensor once; then a few of them again with one activation row
    for start in range(0, cols, 8):
        picked = order[start : start + 8]
        x = np.zeros((8, cols), dtype=np.float32)
        x[np.arange(8), picked] = 1.0
        rt.write("x", x)
        rt.qmv("w", "x", "y", 8)
        rt.synchronize()
        got = rt.read_array("y", 8 * rows).reshape(8, rows)
        # (a sum cannot return -0.0; comparing values treats the two zeros as equal and everything else exactly)
        assert np.array_equal(got, want[:, picked].T), (t.name, start)
    for c in order[:24]:
        x = np.zeros(cols, dtype=np.float32)
        x[c] = 1.0
        rt.write("x", x)
        rt.qmv("w", "x", "y", 1)
        rt.synchronize()
        assert np.array_equal(rt.read_array("y", rows), want[:, c]), (t.name, int(c))


@pytest.mark.parametrize("ntok", [1, 2, 4, 8])
@pytest.mark.parametrize("name,t,rows,cols", LAYER_SET, ids=[entry[0] for entry in LAYER_SET])
def test_mixed_layer_every_tensor_and_row_count(rt, clib, codebooks, name, t, rows, cols, ntok):
    rng = np.random.default_rng(2000 + rows + cols + ntok)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    ref = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(_qmv(rt, raw, t, rows, cols, x), ref) <= REL_L2


@pytest.mark.parametrize("ntok", [1, 8])
@pytest.mark.parametrize("t,rows,cols", IQ_SWEEP, ids=[entry[0].name for entry in IQ_SWEEP])
def test_iq_sweep_every_tensor_at_one_and_eight_rows(rt, clib, codebooks, t, rows, cols, ntok):
    rng = np.random.default_rng(3000 + int(t) + ntok)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    ref = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(_qmv(rt, raw, t, rows, cols, x), ref) <= REL_L2
