"""Pins the CPU oracles (oracle/dequant_np.py, oracle/qmv_oracle.c) to the reference.

(a) the known-answer vectors of the reference's engine/tests/test_gguf_dequant.py:38-194,
(b) outputs of the reference dequantiser on seeded random blocks of every type (tests/golden/dequant_golden.npz),
(c) the reference CPU matvec's outputs (tests/golden/cpu_qwen_golden.npz) with the reference's own
    error allowance (engine/tests/test_phase31e_cpu_layers.py:44-51).
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np
import pytest

from oracle import dequant_np as O
from tests import oracle_libs
from vinf_3080ti_b200.gguf_types import TRAITS, GGUFTensorType as T
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def clib():
    return oracle_libs.load_c_oracle()


def both(clib, codebooks, raw: bytes, t: T, n: int) -> np.ndarray:
    """Dequantise with the numpy and the C oracle, require identical bits, return the values."""
    a = O.dequantize(raw, int(t), n, codebooks)
    b = oracle_libs.c_dequantize(clib, np.frombuffer(raw, dtype=np.uint8), int(t), 1, n, codebooks)
    assert np.array_equal(a, b)
    return a


# ---- (a) known-answer vectors ---------------------------------------------------------------------

def test_q8_0_known_answer(clib, codebooks):  # test_gguf_dequant.py:38-45
    v = both(clib, codebooks, struct.pack("<e32b", 0.5, *range(-16, 16)), T.Q8_0, 32)
    assert v[0] == -8.0 and v[-1] == 7.5


def test_q4_k_known_answer(clib, codebooks):  # test_gguf_dequant.py:54-74
    scales = bytes([1, 2, 3, 4, 0, 1, 2, 3, 5, 6, 7, 8])
    qs = bytes(lo | (hi << 4) for lo, hi in zip(range(16), reversed(range(16))))
    v = both(clib, codebooks, struct.pack("<ee", 0.5, 0.25) + scales + qs * 8, T.Q4_K, 256)
    assert list(v[:4]) == [0.0, 0.5, 1.0, 1.5]
    assert list(v[16:20]) == [0.0, 0.5, 1.0, 1.5]
    assert list(v[32:34]) == [14.75, 13.75]
    assert [v[64], v[96], v[128], v[160], v[192], v[224]] == [-0.5, 29.25, 0.0, 45.0, 0.0, 60.0]


def test_q3_k_known_answer(clib, codebooks):  # test_gguf_dequant.py:76-97
    hmask = bytearray([0xFF] * 32)
    hmask[3] &= ~(1 << 5) & 0xFF
    qs = bytearray([0xFF] * 64)
    qs[32] = 0x00
    low = bytes(k | (k + 8) << 4 for k in range(8))
    block = bytes(hmask) + bytes(qs) + low + bytes([0xE4] * 4) + struct.pack("<e", 0.5)
    v = both(clib, codebooks, block, T.Q3_K, 256)
    expect = {0: -48.0, 3: -48.0, 35: -45.0, 80: -16.5, 128: 0.0, 129: 12.0, 160: 0.0, 163: -5.0, 255: 46.5}
    assert {k: v[k] for k in expect} == expect


def test_iq3_s_grid_known_answer(codebooks):  # test_gguf_dequant.py:99-106
    grid = np.frombuffer(codebooks["iq3s_grid"], dtype=np.uint8).reshape(512, 4)
    assert list(grid[0]) == [1, 1, 1, 1] and list(grid[3]) == [11, 1, 1, 1] and list(grid[5]) == [1, 3, 1, 1]


def test_q2_k_known_answer(clib, codebooks):  # test_gguf_dequant.py:108-125
    scales = bytes((k % 16) | (((7 * k) % 16) << 4) for k in range(16))
    qs = bytes((i * 37 + 11) % 256 for i in range(64))
    v = both(clib, codebooks, scales + qs + struct.pack("<ee", 0.5, 0.25), T.Q2_K, 256)
    expected, idx = [], 0
    for n in range(2):
        q = qs[32 * n : 32 * n + 32]
        for j in range(4):
            for s in range(2):
                sc = scales[idx]
                idx += 1
                for l in range(16):
                    expected.append(0.5 * (sc & 0xF) * ((q[16 * s + l] >> (2 * j)) & 3) - 0.25 * (sc >> 4))
    assert list(v) == expected


def test_q5_k_known_answer(clib, codebooks):  # test_gguf_dequant.py:127-142
    scales = bytes([1, 2, 3, 4, 0, 1, 2, 3, 5, 6, 7, 8])
    qs = bytes(lo | (hi << 4) for lo, hi in zip(range(16), reversed(range(16))))
    block = struct.pack("<ee", 0.5, 0.25) + scales + bytes([0b01010101] * 32) + qs * 8
    v = both(clib, codebooks, block, T.Q5_K, 256)
    assert list(v[:4]) == [8.0, 8.5, 9.0, 9.5]
    assert list(v[32:36]) == [14.75, 13.75, 12.75, 11.75]
    assert [v[64], v[96], v[128], v[160], v[192], v[224]] == [23.5, 29.25, 40.0, 45.0, 56.0, 60.0]


def test_q6_k_known_answer(clib, codebooks):  # test_gguf_dequant.py:144-159
    block = bytes([0x10] * 128) + bytes([0b11100100] * 64) + struct.pack("<16b", *range(1, 17)) + struct.pack("<e", 0.5)
    v = both(clib, codebooks, block, T.Q6_K, 256)
    assert [v[0], v[16], v[32], v[48], v[64], v[80], v[96], v[112]] == [-16.0, -32.0, -24.0, -32.0, 2.5, 3.0, 59.5, 68.0]


def test_iq4_nl_known_answer(clib, codebooks):  # test_gguf_dequant.py:161-167
    qs = bytes(lo | (hi << 4) for lo, hi in zip(range(16), reversed(range(16))))
    v = both(clib, codebooks, struct.pack("<e", 0.5) + qs, T.IQ4_NL, 32)
    assert list(v[:4]) == [-63.5, -52.0, -41.5, -32.5] and list(v[16:20]) == [56.5, 44.5, 34.5, 26.5]


def test_iq4_xs_known_answer(clib, codebooks):  # test_gguf_dequant.py:169-178
    qs = bytes(lo | (hi << 4) for lo, hi in zip(range(16), reversed(range(16)))) * 8
    v = both(clib, codebooks, struct.pack("<eH", 0.5, 0xAAAA) + bytes([0x11] * 4) + qs, T.IQ4_XS, 256)
    assert list(v[:4]) == [-63.5, -52.0, -41.5, -32.5] and list(v[32:36]) == [-63.5, -52.0, -41.5, -32.5]


def test_iq3_s_known_answer(clib, codebooks):  # test_gguf_dequant.py:180-194
    block = struct.pack("<e", 0.5) + bytes(64) + bytes(8) + bytes([1] + [0] * 31) + bytes(4)
    v = both(clib, codebooks, block, T.IQ3_S, 256)
    assert v[0] == -0.5 and list(v[1:4]) == [0.5, 0.5, 0.5] and v[32] == 0.5


def test_f32_f16_known_answer(clib, codebooks):  # test_gguf_dequant.py:28-36
    assert list(both(clib, codebooks, struct.pack("<fff", 1.0, -2.0, 3.5), T.F32, 3)) == [1.0, -2.0, 3.5]
    assert list(both(clib, codebooks, struct.pack("<ee", 1.5, -2.0), T.F16, 2)) == [1.5, -2.0]


# ---- (b) the reference dequantiser's outputs --------------------------------------------------------

def test_sign_table_matches_reference(codebooks):
    assert O.ksigns_iq2xs().tobytes() == codebooks["ksigns_iq2xs"]


@pytest.mark.parametrize("t", sorted(TRAITS), ids=lambda t: t.name)
def test_matches_reference_dequantiser_bit_for_bit(clib, codebooks, t):
    with np.load(GOLDEN / "dequant_golden.npz") as z:
        rows, cols = (int(v) for v in z["shape"])
        raw, want = z[f"raw_{int(t)}"], z[f"val_{int(t)}"]
    got = both(clib, codebooks, raw.tobytes(), t, rows * cols)
    assert np.array_equal(got, want.astype(np.float64))
    assert np.array_equal(got.astype(np.float32).astype(np.float64), got)  # exactly representable in fp32


def test_rejects_bad_shapes():
    with pytest.raises(ValueError):
        O.dequantize(bytes(33), int(T.Q8_0), 32)
    with pytest.raises(ValueError):
        O.dequantize(bytes(34), 2, 32)  # Q4_0 has no kernel


# ---- C oracle == numpy oracle on the matvec and the argmax -----------------------------------------

@pytest.mark.parametrize("t", sorted(TRAITS), ids=lambda t: t.name)
def test_c_matvec_matches_numpy(clib, codebooks, t):
    rng = np.random.default_rng(100 + int(t))
    rows, cols, ntok = 7, 768, 3
    raw = synthetic_blocks(t, rows, cols, rng)
    x = synthetic_activations(ntok, cols, rng)
    a = O.matvec(raw, int(t), rows, cols, x, codebooks)
    b = oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x, codebooks)
    np.testing.assert_allclose(b, a, rtol=1e-12, atol=1e-12 * np.abs(a).max())


def test_argmax_tie_and_empty_rules(clib):
    y = np.array([[1.0, 3.0, 3.0, 2.0], [-np.inf] * 4, [np.nan, -1.0, np.nan, -1.0]])
    assert list(O.argmax_rows(y)) == [1, 0x7FFFFFFF, 1]
    assert list(oracle_libs.c_argmax_rows(clib, y)) == [1, 0x7FFFFFFF, 1]


# ---- (c) the reference CPU matvec -------------------------------------------------------------------

@pytest.mark.parametrize("t", sorted(TRAITS), ids=lambda t: t.name)
def test_reference_cpu_matvec_golden_within_its_bound(codebooks, t):
    with np.load(GOLDEN / "cpu_qwen_golden.npz") as z:
        rows, cols, ntok = (int(v) for v in z["shape"])
        raw, x, y = z[f"raw_{int(t)}"], z[f"x_{int(t)}"], z[f"y_{int(t)}"]
    ref = O.matvec(raw, int(t), rows, cols, x, codebooks)
    if t in (T.F32, T.F16):
        bound = np.zeros_like(ref)
    else:
        bound = O.cpu_qwen_bound(raw, int(t), rows, cols, x, codebooks)
    assert np.all(np.abs(y - ref) <= bound + 1e-4 * (1 + np.abs(ref)))


def test_built_reference_cpu_module_reproduces_its_golden(codebooks):
    mod = oracle_libs.load_reference_cpu_module()
    if mod is None:
        pytest.skip("oracle/_ref is not built (make -C oracle ref REFERENCE=...)")
    rt = mod.CpuRuntime(codebooks["iq3s_grid"], 2)
    with np.load(GOLDEN / "cpu_qwen_golden.npz") as z:
        rows, cols, ntok = (int(v) for v in z["shape"])
        keep = []
        for t in sorted(TRAITS):
            raw, x, y = z[f"raw_{int(t)}"].tobytes(), z[f"x_{int(t)}"], z[f"y_{int(t)}"]
            keep.append(raw)
            name = f"w{int(t)}"
            rt.add_tensor(name, raw, int(t), cols, rows)
            rt.alloc(name + ".x", cols * ntok)
            rt.alloc(name + ".y", rows * ntok)
            rt.write(name + ".x", x.tobytes())
            rt.qmv(name, name + ".x", name + ".y", ntok)
            got = np.frombuffer(rt.read(name + ".y"), dtype=np.float32).reshape(ntok, rows)
            np.testing.assert_allclose(got, y, rtol=1e-6, atol=1e-6)
