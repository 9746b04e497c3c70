"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Bars: dequantised values bit-exact; matvec relative L2 error <= 1e-5 against dequantise + fp64 matvec (and
the reference's own per-element bound 1e-4 * max|ref| + 1e-5, engine/tests/test_phase30_cuda_qmatvec.py:67-72);
argmax ids exact.  Shapes follow the reference's tests (5 x 512 for every type, 70 x 512 with 37 rows of
activations, engine/tests/test_phase31i_prefill.py:194-219) plus ragged and benchmark-sized ones.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

from oracle import dequant_np as O
from tests import oracle_libs
from vinf_3080ti_b200.gguf_types import TRAITS, GGUFTensorType as T
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
ALL_TYPES = sorted(TRAITS)
REL_L2 = 1e-5  # fp32 accumulation, stated by the task


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


def run_qmv(rt, raw: np.ndarray, t: T, rows: int, cols: int, x: np.ndarray, name: str = "w") -> np.ndarray:
    ntok = x.shape[0]
    rt.upload(name, raw, int(t), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", np.ascontiguousarray(x, dtype=np.float32))
    rt.qmv(name, "x", "y", ntok)
    rt.synchronize()
    return rt.read_array("y").reshape(ntok, rows).copy()


# ---- dequantised values: bit-exact ------------------------------------------------------------------

@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_dequantised_values_equal_the_reference_dequantiser(rt, t):
    with np.load(GOLDEN / "dequant_golden.npz") as z:
        rows, cols = (int(v) for v in z["shape"])
        raw, want = z[f"raw_{int(t)}"], z[f"val_{int(t)}"]
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("deq", rows * cols)
    rt.dequantize("w", "deq")
    rt.synchronize()
    got = rt.read_array("deq")
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_dequantised_values_bit_exact_on_benchmark_width_rows(rt, codebooks, t):
    rng = np.random.default_rng(500 + int(t))
    rows, cols = 64, 5120
    raw = synthetic_blocks(t, rows, cols, rng)
    want = O.dequantize(raw, int(t), rows * cols, codebooks).astype(np.float32)
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("deq", rows * cols)
    rt.dequantize("w", "deq")
    rt.synchronize()
    assert np.array_equal(rt.read_array("deq").view(np.uint32), want.view(np.uint32))


# ---- matvec ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_matvec_entry_on_the_reference_test_shape(rt, codebooks, t):
    """5 x 512, one activation row, through the synchronous matvec entry (test_phase30_cuda_qmatvec.py:74-86)."""
    rng = np.random.default_rng(30 + int(t))
    rows, cols = 5, 512
    raw = synthetic_blocks(t, rows, cols, rng, 0.001, 0.05)
    x = rng.uniform(-1, 1, cols).astype(np.float32)
    rt.upload("w", raw, int(t), cols, rows)
    got = np.frombuffer(rt.matvec("w", x), dtype=np.float32)
    ref = O.matvec(raw, int(t), rows, cols, x, codebooks)
    assert np.all(np.isfinite(got))
    assert np.all(np.abs(got - ref) <= 1e-4 * max(1e-6, np.abs(ref).max()) + 1e-5)
    assert rel_l2(got, ref) <= REL_L2
    rt.free("w")
    assert rt.device_bytes() == 0


@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
@pytest.mark.parametrize("ntok", [1, 2, 3, 4, 5, 6, 7, 8])
def test_qmv_every_type_and_row_count(rt, codebooks, t, ntok):
    rng = np.random.default_rng(1000 + 16 * int(t) + ntok)
    rows, cols = 70, 1536  # rows not a multiple of the row-group height; one full and one half segment
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    got = run_qmv(rt, raw, t, rows, cols, x)
    ref = O.matvec(raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, ref) <= REL_L2


@pytest.mark.parametrize("t,rows,cols", [
    (T.Q8_0, 3, 32), (T.IQ4_NL, 1, 32), (T.F32, 9, 32), (T.F16, 2, 64), (T.Q4_K, 1, 256), (T.Q6_K, 7, 256),
    (T.Q3_K, 1025, 768), (T.IQ2_XXS, 33, 2304), (T.Q5_K, 300, 1024), (T.Q2_K, 5, 4352), (T.IQ4_XS, 129, 5120),
], ids=lambda v: getattr(v, "name", str(v)))
def test_qmv_ragged_and_minimal_shapes(rt, codebooks, t, rows, cols):
    rng = np.random.default_rng(rows * 7919 + cols)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(3, cols, rng)
    got = run_qmv(rt, raw, t, rows, cols, x)
    ref = O.matvec(raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, ref) <= REL_L2


@pytest.mark.parametrize("t", [T.Q4_K, T.Q6_K, T.Q3_K, T.IQ4_XS, T.IQ2_S, T.Q8_0], ids=lambda t: t.name)
def test_batched_pass_equals_single_row_passes_bit_for_bit(rt, t):
    """engine/tests/test_phase31c_batched_forward.py:53-66 at the matvec level."""
    rng = np.random.default_rng(31 + int(t))
    rows, cols, ntok = 300, 2048, 8
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    together = run_qmv(rt, raw, t, rows, cols, x)
    for k in range(ntok):
        alone = run_qmv(rt, raw, t, rows, cols, x[k : k + 1])
        assert np.array_equal(alone[0].view(np.uint32), together[k].view(np.uint32))


@pytest.mark.parametrize("t", [T.Q4_K, T.Q6_K], ids=lambda t: t.name)
def test_wide_pass_runs_as_groups_of_eight(rt, codebooks, t):
    """70 x 512 weights, 37 activation rows: partial last group (test_phase31i_prefill.py:194-219)."""
    rng = np.random.default_rng(37)
    rows, cols, ntok = 70, 512, 37
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    got = run_qmv(rt, raw, t, rows, cols, x)
    ref = O.matvec(raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, ref) <= REL_L2


@pytest.mark.parametrize("t,rows,cols,ntok", [
    (T.Q4_K, 17408, 5120, 1), (T.Q4_K, 17408, 5120, 8), (T.Q4_K, 5120, 17408, 4), (T.Q3_K, 17408, 5120, 4),
    (T.Q6_K, 6144, 5120, 2), (T.Q6_K, 1024, 5120, 1), (T.Q6_K, 5120, 6144, 8), (T.IQ4_XS, 17408, 5120, 1),
    (T.IQ2_XXS, 17408, 5120, 8), (T.IQ2_S, 17408, 5120, 1), (T.IQ3_S, 17408, 5120, 8), (T.IQ4_NL, 5120, 17408, 1),
], ids=lambda v: getattr(v, "name", str(v)))
def test_qmv_benchmark_shapes(rt, clib, codebooks, t, rows, cols, ntok):
    rng = np.random.default_rng(0)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    got = run_qmv(rt, raw, t, rows, cols, x)
    ref = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, ref) <= REL_L2


def test_linearity_at_full_size(rt):
    """Size-independent property: W(a*x1 + x2) = a*W x1 + W x2 up to fp32 rounding, no oracle needed."""
    rng = np.random.default_rng(5)
    rows, cols = 17408, 5120
    raw = synthetic_blocks(T.Q4_K, rows, cols, rng)
    x = synthetic_activations(2, cols, rng)
    combo = (2.0 * x[0] + x[1])[None, :]
    y = run_qmv(rt, raw, T.Q4_K, rows, cols, np.concatenate([x, combo]))
    ref = 2.0 * y[0].astype(np.float64) + y[1]
    assert rel_l2(y[2], ref) <= 1e-5


# ---- argmax --------------------------------------------------------------------------------------------

def test_argmax_rows_rules(rt):
    n, ntok = 1000, 5
    rng = np.random.default_rng(9)
    y = rng.standard_normal((ntok, n)).astype(np.float32)
    y[1, 17] = y[1, 900] = 50.0  # tie -> lowest index
    y[2, :] = -np.inf  # nothing above -inf -> 0x7fffffff
    y[3, :] = np.nan
    y[3, 5] = -3.0
    y[4, 999] = 99.0
    rt.alloc("logits", ntok * n)
    rt.write("logits", y)
    assert rt.argmax_rows("logits", n, ntok) == [int(v) for v in O.argmax_rows(y)]
    assert rt.argmax_rows("logits", n, ntok)[1:4] == [17, 0x7FFFFFFF, 5]
    assert rt.argmax("logits", n) == int(np.argmax(y[0]))
    with pytest.raises(ValueError):
        rt.argmax_rows("logits", n, 257)


@pytest.mark.parametrize("t,ntok", [(T.Q6_K, 1), (T.Q6_K, 4), (T.Q4_K, 8), (T.IQ4_XS, 3)], ids=lambda v: getattr(v, "name", str(v)))
def test_fused_lm_head_argmax_matches_unfused_and_oracle(rt, codebooks, t, ntok):
    rng = np.random.default_rng(77 + ntok)
    rows, cols = 4099, 1024
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    ref = O.matvec(raw, int(t), rows, cols, x, codebooks)
    top2 = np.sort(ref, axis=1)[:, -2:]
    assert np.all(top2[:, 1] - top2[:, 0] > 1e-4 * np.abs(top2[:, 1])), "near-tie in the synthetic logits: reseed"
    logits = run_qmv(rt, raw, t, rows, cols, x)
    unfused = rt.argmax_rows("y", rows, ntok)
    rt.alloc("y2", ntok * rows)
    fused = rt.qmv_argmax("w", "x", "y2", ntok)
    assert fused == unfused == [int(v) for v in O.argmax_rows(ref)]
    assert np.array_equal(rt.read_array("y2").view(np.uint32), logits.reshape(-1).view(np.uint32))
    assert rt.qmv_argmax("w", "x", None, ntok) == fused  # without storing the logits
    rt.qmv_argmax("w", "x", None, ntok, blocking=False)  # ids stay on the device; twice in a row works
    assert rt.qmv_argmax("w", "x", None, ntok) == fused


def test_fused_argmax_ties_go_to_the_lowest_row(rt):
    rows, cols = 515, 256
    w = np.zeros((rows, cols), dtype=np.float32)
    w[[7, 300, 514], 0] = 2.0  # three equal maxima
    w[100, 0] = -1.0
    x = np.zeros((2, cols), dtype=np.float32)
    x[0, 0] = 1.0
    x[1, 0] = -1.0  # second row: maximum is row 100's +1
    rt.upload("w", w, int(T.F32), cols, rows)
    rt.alloc("x", 2 * cols)
    rt.write("x", x)
    assert rt.qmv_argmax("w", "x", None, 2) == [7, 100]


# ---- boundary behaviour --------------------------------------------------------------------------------

def test_error_contract(rt):
    """engine/tests/test_phase30_cuda_qmatvec.py:127-134 and the checks of Runtime_qmv / find_buffer."""
    with pytest.raises(ValueError):
        rt.upload("w", bytes(34), 2, 32, 1)  # Q4_0: no kernel
    with pytest.raises(ValueError):
        rt.upload("w", bytes(33), int(T.Q8_0), 32, 1)  # wrong byte count
    with pytest.raises(ValueError):
        rt.upload("w", bytes(144), int(T.Q4_K), 100, 1)  # cols not a multiple of the block
    with pytest.raises(KeyError):
        rt.matvec("missing", np.zeros(32, dtype=np.float32))
    with pytest.raises(KeyError):
        rt.free("missing")
    rt.upload("w8", bytes(34 * 2), int(T.Q8_0), 32, 2)
    rt.alloc("x", 32)
    rt.alloc("y", 2)
    with pytest.raises(KeyError):
        rt.qmv("nope", "x", "y")
    with pytest.raises(KeyError):
        rt.qmv("w8", "nope", "y")
    with pytest.raises(ValueError):
        rt.qmv("w8", "x", "y", 0)
    with pytest.raises(ValueError):
        rt.qmv("w8", "x", "y", 2)  # buffers too small for two rows
    rt.alloc("h", 64, 2)
    with pytest.raises(TypeError):
        rt.qmv("w8", "h", "y")
    with pytest.raises(ValueError):
        rt.alloc("bad", 0)
    with pytest.raises(ValueError):
        rt.alloc("bad", 4, 3)
    with pytest.raises(ValueError):
        rt.write("x", bytes(4 * 33))
    with pytest.raises(ValueError):
        rt.read("x", 33)
    assert rt.has("w8") and not rt.has("nope")
    addr, typ, rows, cols, row_bytes, nbytes, resident = rt.tensor_info("w8")
    assert (typ, rows, cols, row_bytes, nbytes, resident) == (8, 2, 32, 34, 68, True) and addr % 256 == 0


def test_buffers_copy_zero_and_reupload(rt):
    rt.alloc("a", 16)
    rt.alloc("b", 16)
    rt.write("a", np.arange(16, dtype=np.float32))
    rt.copy("b", 4, "a", 8, 4)
    rt.synchronize()
    assert list(rt.read_array("b")[4:8]) == [8.0, 9.0, 10.0, 11.0] and rt.read_array("b")[0] == 0.0
    rt.zero_range("a", 2, 3)
    rt.synchronize()
    assert list(rt.read_array("a")[:6]) == [0.0, 1.0, 0.0, 0.0, 0.0, 5.0]
    rt.zero("a")
    assert not rt.read_array("a").any()
    assert rt.read("a", 2, 14) == bytes(8)
    rt.alloc("a", 4)  # re-alloc replaces
    assert rt.buffer_ptr("a")[1] == 4


def test_codebook_must_be_set_before_use():
    from vinf_3080ti_b200.runtime import Runtime

    bare = Runtime()
    rng = np.random.default_rng(1)
    bare.upload("w", synthetic_blocks(T.IQ2_XS, 2, 256, rng), int(T.IQ2_XS), 256, 2)
    bare.alloc("x", 256)
    bare.alloc("y", 2)
    with pytest.raises(ValueError, match="codebook"):
        bare.qmv("w", "x", "y")
    bare.close()


def test_a_captured_pass_replays_as_one_graph(rt, codebooks):
    rng = np.random.default_rng(12)
    shapes = [(T.Q6_K, 96, 512), (T.Q3_K, 200, 512), (T.Q4_K, 512, 768)]
    raws = [synthetic_blocks(t, r, c, rng) for t, r, c in shapes]
    for i, ((t, r, c), raw) in enumerate(zip(shapes, raws)):
        rt.upload(f"g{i}", raw, int(t), c, r)
        rt.alloc(f"gy{i}", 2 * r)
    x = synthetic_activations(2, 512, rng)
    x3 = synthetic_activations(2, 768, rng)
    rt.alloc("gx", 2 * 512)
    rt.alloc("gx3", 2 * 768)
    rt.write("gx", x)
    rt.write("gx3", x3)
    before = rt.launch_count()
    rt.capture_begin()
    rt.qmv("g0", "gx", "gy0", 2)
    rt.qmv("g1", "gx", "gy1", 2)
    rt.qmv("g2", "gx3", "gy2", 2)
    with pytest.raises(ValueError):
        rt.read("gy0")  # blocking calls are refused during capture
    graph = rt.capture_end()
    assert rt.launch_count() == before  # nothing ran yet
    rt.graph_launch(graph)
    rt.synchronize()
    assert rt.launch_count() == before + 3
    for i, ((t, r, c), raw) in enumerate(zip(shapes, raws)):
        ref = O.matvec(raw, int(t), r, c, x3 if c == 768 else x, codebooks)
        assert rel_l2(rt.read_array(f"gy{i}").reshape(2, r), ref) <= REL_L2
    rt.graph_destroy(graph)


# ---- prompt-pass GEMM (tensor cores) --------------------------------------------------------------------------

@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_prompt_gemm_matches_the_matvec_path_for_every_type(rt, codebooks, t):
    """engine/tests/test_phase31i_prefill.py:194-219: 70 x 512 weights, 37 activation rows (partial tiles), fp16
    operands, tolerance 3e-3 * max|ref| against the fp32 matvec groups."""
    rng = np.random.default_rng(3100 + int(t))
    rows, cols, ntok = 70, 512, 37
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    ref = run_qmv(rt, raw, t, rows, cols, x)  # fp32 matvec, groups of 8
    rt.set_gemm_min_rows(1)
    try:
        rt.zero("y")
        rt.qmv("w", "x", "y", ntok)
        rt.synchronize()
        got = rt.read_array("y").reshape(ntok, rows)
    finally:
        rt.set_gemm_min_rows(0)
    assert np.all(np.abs(got - ref) <= 3e-3 * np.abs(ref).max())
    oracle = O.matvec(raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, oracle) <= 2e-3  # fp16 rounding of both operands


@pytest.mark.parametrize("t,rows,cols,ntok", [(T.Q4_K, 1000, 5120, 512), (T.Q6_K, 321, 1024, 300), (T.IQ3_S, 64, 768, 256)],
                         ids=lambda v: getattr(v, "name", str(v)))
def test_prompt_gemm_larger_shapes_and_threshold(rt, clib, codebooks, t, rows, cols, ntok):
    rng = np.random.default_rng(rows + ntok)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", x)
    rt.set_gemm_min_rows(64)
    try:
        rt.qmv("w", "x", "y", ntok)  # >= 64 rows: GEMM
        rt.synchronize()
        got = rt.read_array("y").reshape(ntok, rows).copy()
        rt.qmv("w", "x", "y", 8)  # below the threshold: still the fp32 matvec
        rt.synchronize()
        small = rt.read_array("y", 8 * rows).reshape(8, rows)
    finally:
        rt.set_gemm_min_rows(0)
    ref = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, ref) <= 2e-3
    assert rel_l2(small, ref[:8]) <= REL_L2
    with pytest.raises(ValueError):
        rt.set_gemm_min_rows(-1)


# ---- several tensors in one launch; short launches split by columns ------------------------------------------

def _upload_group(rt, t, shapes, cols, ntok, rng):
    raws = []
    for i, rows in enumerate(shapes):
        raw = synthetic_blocks(t, rows, cols, rng)
        rt.upload(f"g{i}", raw, int(t), cols, rows)
        rt.alloc(f"gy{i}", ntok * rows)
        rt.alloc(f"sy{i}", ntok * rows)
        raws.append(raw)
    return raws


@pytest.mark.parametrize("t,shapes,ntok", [(T.Q6_K, (1538, 258, 256), 4), (T.Q3_K, (2048, 2050), 1), (T.Q4_K, (1301, 77, 300, 5), 8),
                                            (T.IQ4_XS, (1400, 3), 3), (T.IQ3_S, (1500, 700), 2)], ids=lambda v: getattr(v, "name", str(v)))
def test_group_launch_equals_one_launch_per_tensor_bit_for_bit(rt, codebooks, t, shapes, ntok):
    """q/k/v-like and gate/up-like groups: one launch over all rows gives every tensor exactly what its own launch
    gives, as long as short launches are not split by columns (the short tensors' own launches would be)."""
    rng = np.random.default_rng(sum(shapes) + ntok)
    cols = 1024
    raws = _upload_group(rt, t, shapes, cols, ntok, rng)
    x = synthetic_activations(ntok, cols, rng)
    rt.alloc("x", ntok * cols)
    rt.write("x", x)
    n = len(shapes)
    rt.set_column_split(False)
    try:
        rt.qmv_group([f"g{i}" for i in range(n)], "x", [f"gy{i}" for i in range(n)], ntok)
        for i in range(n):
            rt.qmv(f"g{i}", "x", f"sy{i}", ntok)
        rt.synchronize()
    finally:
        rt.set_column_split(True)
    for i, rows in enumerate(shapes):
        grouped = rt.read_array(f"gy{i}", ntok * rows)
        assert np.array_equal(grouped.view(np.uint32), rt.read_array(f"sy{i}", ntok * rows).view(np.uint32)), i
        ref = O.matvec(raws[i], int(t), rows, cols, x, codebooks)
        assert rel_l2(grouped.reshape(ntok, rows), ref) <= REL_L2


@pytest.mark.parametrize("t,shapes,cols,ntok", [(T.Q6_K, (768, 128, 128), 5120, 4), (T.Q4_K, (640,), 17408, 4), (T.Q3_K, (90, 30), 3072, 8),
                                                 (T.Q6_K, (9,), 5120, 1), (T.IQ2_S, (400, 200), 2304, 2), (T.Q8_0, (1184,), 2048, 3)],
                         ids=lambda v: getattr(v, "name", str(v)))
def test_short_launches_split_by_columns_match_the_oracle(rt, clib, codebooks, t, shapes, cols, ntok):
    """Row shards of an 8-GPU split and other short launches: the rows' columns are shared among several blocks whose
    partial sums are added in column order.  Same tolerance as everywhere, and an M-row pass still equals M single-row
    passes bit for bit."""
    rng = np.random.default_rng(sum(shapes) + cols + ntok)
    raws = _upload_group(rt, t, shapes, cols, ntok, rng)
    x = synthetic_activations(ntok, cols, rng)
    rt.alloc("x", ntok * cols)
    rt.alloc("x1", cols)
    rt.write("x", x)
    n = len(shapes)
    names, outs = [f"g{i}" for i in range(n)], [f"gy{i}" for i in range(n)]
    rt.qmv_group(names, "x", outs, ntok)
    rt.synchronize()
    got = [rt.read_array(f"gy{i}", ntok * rows).reshape(ntok, rows).copy() for i, rows in enumerate(shapes)]
    for i, rows in enumerate(shapes):
        ref = oracle_libs.c_qmv(clib, raws[i], int(t), rows, cols, x, codebooks)
        assert rel_l2(got[i], ref) <= REL_L2, i
    for k in range(ntok):
        rt.write("x1", x[k])
        rt.qmv_group(names, "x1", outs, 1)
        rt.synchronize()
        for i, rows in enumerate(shapes):
            assert np.array_equal(rt.read_array(f"gy{i}", rows).view(np.uint32), got[i][k].view(np.uint32)), (i, k)


def test_group_launch_error_contract(rt):
    rng = np.random.default_rng(5)
    rt.upload("ga", synthetic_blocks(T.Q6_K, 7, 256, rng), int(T.Q6_K), 256, 7)   # 7 rows of 210 bytes: the next tensor's rows
    rt.upload("gb", synthetic_blocks(T.Q6_K, 8, 256, rng), int(T.Q6_K), 256, 8)   # would start at byte 14 of a 16-byte line, not at 0
    rt.upload("gc", synthetic_blocks(T.Q4_K, 8, 256, rng), int(T.Q4_K), 256, 8)
    rt.upload("gd", synthetic_blocks(T.Q6_K, 8, 512, rng), int(T.Q6_K), 512, 8)
    for name, n in (("x", 8 * 512), ("ya", 64), ("yb", 64), ("small", 4)):
        rt.alloc(name, n)
    rt.qmv_group(["gb", "ga"], "x", ["yb", "ya"], 2)  # 8 rows first: fine
    rt.synchronize()
    with pytest.raises(ValueError):
        rt.qmv_group(["ga", "gb"], "x", ["ya", "yb"], 2)
    with pytest.raises(ValueError):
        rt.qmv_group(["gb", "gc"], "x", ["ya", "yb"], 1)  # types differ
    with pytest.raises(ValueError):
        rt.qmv_group(["gb", "gd"], "x", ["ya", "yb"], 1)  # columns differ
    with pytest.raises(ValueError):
        rt.qmv_group(["gb"] * 5, "x", ["ya"] * 5, 1)
    with pytest.raises(ValueError):
        rt.qmv_group(["gb"], "x", ["small"], 1)
    with pytest.raises(KeyError):
        rt.qmv_group(["gb", "nope"], "x", ["ya", "yb"], 1)
    with pytest.raises(ValueError):
        rt.qmv_group(["gb"], "x", ["ya"], 9)


@pytest.mark.parametrize("rows,ntok", [(200, 130), (300, 300), (200, 700)], ids=lambda v: str(v))
@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_prompt_gemm_tcgen05_matches_the_matvec_path_for_every_type(rt, codebooks, t, rows, ntok):
    """Passes of 64+ activation rows take the tcgen05 kernel (accumulators in tensor memory), in each of its block shapes:
    up to 256 activation rows (one accumulator per block); more than that (two accumulators: 256 weight rows per block,
    or 512 activation rows for the types whose raw blocks for 256 rows do not fit in shared memory); several tiles of
    activation rows.  The weight rows end inside a tile, and inside its first half.  Same tolerance as the warp-level
    kernel."""
    rng = np.random.default_rng(5100 + int(t) + ntok)
    cols = 1024
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    ref = run_qmv(rt, raw, t, rows, cols, x)  # fp32 matvec, groups of 8
    rt.set_gemm_min_rows(64)
    try:
        rt.zero("y")
        rt.qmv("w", "x", "y", ntok)
        rt.synchronize()
        got = rt.read_array("y").reshape(ntok, rows)
    finally:
        rt.set_gemm_min_rows(0)
    assert np.all(np.abs(got - ref) <= 3e-3 * np.abs(ref).max())
    oracle = O.matvec(raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, oracle) <= 2e-3  # fp16 rounding of both operands


@pytest.mark.parametrize("ntok", [130, 300])
@pytest.mark.parametrize("t", [T.Q8_0, T.IQ4_NL, T.F16, T.F32], ids=lambda t: t.name)
def test_prompt_gemm_tcgen05_columns_that_end_inside_a_run_of_256(rt, codebooks, t, ntok):
    """Types with blocks of 32 weights (or none) allow column counts that are not multiples of 256: the kernel's last run of
    raw blocks is then short (320 columns: one full run and a quarter of one)."""
    rng = np.random.default_rng(7300 + int(t) + ntok)
    rows, cols = 150, 320
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    ref = run_qmv(rt, raw, t, rows, cols, x)
    rt.set_gemm_min_rows(64)
    try:
        rt.zero("y")
        rt.qmv("w", "x", "y", ntok)
        rt.synchronize()
        got = rt.read_array("y").reshape(ntok, rows)
    finally:
        rt.set_gemm_min_rows(0)
    assert np.all(np.abs(got - ref) <= 3e-3 * np.abs(ref).max())


@pytest.mark.parametrize("ntok", [256, 512])
@pytest.mark.parametrize("t", ALL_TYPES, ids=lambda t: t.name)
def test_prompt_gemm_tiles_hold_the_dequantised_weights_rounded_to_fp16(rt, codebooks, t, ntok):
    """One-hot activation rows read the fp16 weight tiles of the tcgen05 kernel back: activation row k = unit vector k
    makes output [k][row] the weight [row][k] as the kernel's producers stored it.  It must be the exact dequantised value
    rounded to fp16 (to nearest even), for the generic decoders and for the fast per-block ones alike, in the block
    shapes for up to 256 and for more activation rows."""
    rng = np.random.default_rng(6200 + int(t))
    rows, cols = 300, 512
    raw = synthetic_blocks(t, rows, cols, rng)
    x = np.zeros((ntok, cols), dtype=np.float32)
    x[np.arange(ntok), np.arange(ntok)] = 1.0
    rt.upload("w", raw, int(t), cols, rows)
    rt.alloc("x", ntok * cols)
    rt.alloc("y", ntok * rows)
    rt.write("x", x)
    rt.set_gemm_min_rows(64)
    try:
        rt.qmv("w", "x", "y", ntok)
        rt.synchronize()
        got = rt.read_array("y").reshape(ntok, rows)
    finally:
        rt.set_gemm_min_rows(0)
    w = O.dequantize(raw, int(t), rows * cols, codebooks).reshape(rows, cols)
    with np.errstate(over="ignore"):
        want = w[:, :ntok].astype(np.float16).astype(np.float32).T
    finite = np.isfinite(want)  # synthetic F32 / F16 values beyond the fp16 range would be inf in the tile
    assert finite.mean() > 0.99
    assert np.array_equal(got[finite], want[finite])


@pytest.mark.parametrize("t,rows,cols,ntok", [
    (T.Q6_K, 12288, 5120, 4), (T.Q5_K, 10240, 5120, 1), (T.Q8_0, 6144, 5120, 8), (T.Q8_0, 48, 5120, 4), (T.F32, 48, 5120, 3),
    (T.Q5_K, 5120, 6144, 4), (T.F16, 256, 5120, 2), (T.Q6_K, 19000, 5120, 5), (T.Q4_K, 641, 17408, 7),
], ids=lambda v: getattr(v, "name", str(v)))
def test_qmv_real_model_shapes(rt, clib, codebooks, t, rows, cols, ntok):
    """Shapes of the real 27B tensor set that the synthetic layer set leaves out (engine/src/vinf/gguf/qwen_tensors.py:108-118):
    the gated 12288-row q, the SSM projections of 10240 / 6144 / 48 rows with their Q5_K / Q8_0 / F32 types, an LM-head
    shard, and an odd-sized shard of the down projection."""
    rng = np.random.default_rng(rows + cols + ntok)
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    got = run_qmv(rt, raw, t, rows, cols, x)
    ref = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
    assert rel_l2(got, ref) <= REL_L2


def test_a_graph_that_captured_a_prompt_pass_pins_the_activation_buffer(rt, codebooks):
    """A captured prompt pass holds the address of the runtime's fp16 activation buffer: a wider pass that would have to
    replace that buffer is refused until the graph is destroyed."""
    rng = np.random.default_rng(77)
    rows, cols = 96, 8192  # 1024 x 8192 activations: more than any earlier prompt pass of this module has sized the buffer for
    rt.upload("w", synthetic_blocks(T.Q4_K, rows, cols, rng), int(T.Q4_K), cols, rows)
    rt.alloc("x", 1024 * cols)
    rt.alloc("y", 1024 * rows)
    rt.set_gemm_min_rows(64)
    try:
        rt.qmv("w", "x", "y", 64)  # sizes the buffer for 64 rows
        rt.synchronize()
        rt.capture_begin()
        rt.qmv("w", "x", "y", 64)
        graph = rt.capture_end()
        with pytest.raises(ValueError, match="captured graph"):
            rt.qmv("w", "x", "y", 1024)
        rt.graph_launch(graph)  # still valid
        rt.synchronize()
        rt.graph_destroy(graph)
        rt.qmv("w", "x", "y", 1024)  # now the buffer may grow
        rt.synchronize()
    finally:
        rt.set_gemm_min_rows(0)


def test_issue_rate_probe_reports_plausible_rates():
    """The probe behind the instruction-issue roofline: every kind costs between half a cycle and a few cycles per warp
    instruction, and the decode sequence of 8 weights costs more with 4 activation rows than with 1."""
    from vinf_3080ti_b200.runtime import PROBE_KINDS, probe_issue_rates

    rates = probe_issue_rates(16)
    assert list(rates) == list(PROBE_KINDS)
    for kind in PROBE_KINDS[:8]:
        assert 0.4 <= rates[kind] <= 8.0, (kind, rates[kind])
    assert 8.0 <= rates[PROBE_KINDS[8]] < rates[PROBE_KINDS[9]] <= 200.0
    with pytest.raises(ValueError):
        probe_issue_rates(5)
