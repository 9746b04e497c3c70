"""The matvec with fused prologues / epilogues (Runtime.qmv_fused) against the oracle's double-precision formulas of the same
flags (engine/csrc/megakernel/qwen_megakernel.cu:486-550 for the activations, :231 for the residual add, :233-236 and
:800-829 for the argmax): silu(x) * x2, rmsnorm times its weights, y += W v, argmax over the stored values."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import dequant_np as O
from vinf_3080ti_b200.gguf_types import GGUFTensorType as T
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu
REL_L2 = 1e-5


@pytest.fixture(scope="module")
def rt(codebooks):
    from vinf_3080ti_b200.runtime import Runtime

    runtime = Runtime(codebooks["iq3s_grid"], codebooks)
    yield runtime
    runtime.close()


def rel_l2(got, ref):
    return float(np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref))


CASES = [  # type, rows, cols, ntok, silu_mul, norm, add
    (T.Q4_K, 300, 2048, 1, False, True, False),   # the q/k/v and gate/up projections: rmsnorm on the way in
    (T.Q6_K, 129, 5120, 4, False, True, True),
    (T.Q4_K, 96, 1536, 3, True, False, True),     # the down projection: silu(gate) * up on the way in, residual on the way out
    (T.Q3_K, 5000, 1024, 2, True, True, False),   # both prologues; tall enough for several rows per warp
    (T.IQ4_XS, 70, 768, 8, False, False, True),   # the residual add alone
    (T.Q6_K, 9, 5120, 1, True, True, True),       # a short launch, split by columns over a cluster
    (T.Q8_0, 40, 1056, 5, True, True, True),      # columns not a multiple of 256: a ragged last segment
]


@pytest.mark.parametrize("t,rows,cols,ntok,silu,norm,add", CASES, ids=lambda v: getattr(v, "name", str(v)))
def test_fused_prologues_and_residual_match_the_formulas(rt, codebooks, t, rows, cols, ntok, silu, norm, add):
    rng = np.random.default_rng(rows * 31 + cols + ntok)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    x2 = synthetic_activations(ntok, cols, rng) if silu else None
    nw = rng.uniform(0.5, 1.5, cols).astype(np.float32) if norm else None
    res = (100.0 * rng.standard_normal((ntok, rows))).astype(np.float32) if add else None
    eps = 1e-6
    ref = O.fused_matvec(raw, int(t), rows, cols, x, codebooks, x2=x2, norm_w=nw, eps=eps, residual=res)
    rt.upload("w", raw, int(t), cols, rows)
    for name, n in (("x", ntok * cols), ("x2", ntok * cols), ("nw", cols), ("y", ntok * rows)):
        rt.alloc(name, n)
    rt.write("x", x)
    if silu:
        rt.write("x2", x2)
    if norm:
        rt.write("nw", nw)
    if add:
        rt.write("y", res)
    rt.qmv_fused("w", "x", "y", ntok, add=add, norm="nw" if norm else None, eps=eps, silu_mul="x2" if silu else None)
    rt.synchronize()
    got = rt.read_array("y").reshape(ntok, rows)
    # with a residual the reference value is dominated by it: measure the error on the matvec's own contribution
    own, own_ref = (got.astype(np.float64) - res, ref - res) if add else (got, ref)
    assert rel_l2(np.asarray(own), own_ref) <= (2e-5 if add else REL_L2)  # (the fp32 add of a large residual rounds the sum)
    assert np.array_equal(rt.read_array("x").reshape(ntok, cols), x)  # the inputs are left as they were


def test_fused_flags_leave_the_plain_matvec_bit_identical(rt):
    rng = np.random.default_rng(8)
    rows, cols, ntok = 400, 2048, 4
    raw = synthetic_blocks(T.Q4_K, rows, cols, rng)
    rt.upload("w", raw, int(T.Q4_K), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.alloc("y2", ntok * rows)
    rt.write("x", synthetic_activations(ntok, cols, rng))
    rt.qmv("w", "x", "y", ntok)
    rt.qmv_fused("w", "x", "y2", ntok)  # no flag set
    rt.synchronize()
    assert np.array_equal(rt.read_array("y").view(np.uint32), rt.read_array("y2").view(np.uint32))


def test_lm_head_with_norm_and_argmax_in_one_launch(rt, codebooks):
    """The reference's megakernel LM head: qmv(..., flags = NORM | ARGMAX) (engine/src/vinf/qwen_megakernel.py:341-344)."""
    rng = np.random.default_rng(21)
    rows, cols, ntok = 4099, 1024, 3
    raw = synthetic_blocks(T.Q6_K, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    nw = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    ref = O.fused_matvec(raw, int(T.Q6_K), rows, cols, x, codebooks, norm_w=nw, eps=1e-6)
    top2 = np.sort(ref, axis=1)[:, -2:]
    assert np.all(top2[:, 1] - top2[:, 0] > 1e-4 * np.abs(top2[:, 1])), "near-tie in the synthetic logits: reseed"
    rt.upload("w", raw, int(T.Q6_K), cols, rows)
    rt.upload("nw_tensor", nw, int(T.F32), cols, 1)  # the reference keeps norm weights as one-dimensional F32 tensors
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", x)
    before = rt.launch_count()
    ids = rt.qmv_fused("w", "x", "y", ntok, norm="nw_tensor", eps=1e-6, argmax=True)
    assert rt.launch_count() == before + 1  # rmsnorm, matvec and argmax: one launch
    assert ids == [int(v) for v in O.argmax_rows(ref)]
    assert rel_l2(rt.read_array("y").reshape(ntok, rows), ref) <= REL_L2
    assert rt.qmv_fused("w", "x", None, ntok, norm="nw_tensor", eps=1e-6, argmax=True) == ids  # ids only


def test_fused_error_contract(rt):
    rng = np.random.default_rng(3)
    rt.upload("w", synthetic_blocks(T.Q4_K, 8, 256, rng), int(T.Q4_K), 256, 8)
    rt.alloc("x", 256)
    rt.alloc("y", 8)
    rt.alloc("short", 100)
    with pytest.raises(KeyError):
        rt.qmv_fused("w", "x", "y", 1, norm="nope")
    with pytest.raises(ValueError):
        rt.qmv_fused("w", "x", "y", 1, norm="short")  # fewer norm weights than columns
    with pytest.raises(ValueError):
        rt.qmv_fused("w", "x", "y", 1, silu_mul="short")
    with pytest.raises(ValueError):
        rt.qmv_fused("w", "x", None, 1, add=True, argmax=True)  # a residual needs y
    with pytest.raises(ValueError):
        rt.qmv_fused("w", "x", "y", 9)
