"""TEST INFRASTRUCTURE ONLY - CPU oracle for the quantized matvec path (numpy).

A vectorised restatement of the reference's double-precision block dequantiser
(engine/src/vinf/gguf/dequant.py:121-500) and of its matvec / argmax checks
(engine/src/vinf/reference_ops.py:18-32, engine/csrc/megakernel/qwen_runtime.cu:851-876).
Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
shipped library never does.

Parity status: PINNED.  tests/test_oracle_golden.py checks every function here against
(a) the known-answer vectors of the reference's engine/tests/test_gguf_dequant.py and
(b) outputs of the reference dequantiser itself on seeded random blocks of all 15 types,
stored in tests/golden/dequant_golden.npz by tests/golden/make_golden.py.

Every product that occurs in dequantisation (fp16 scale x small integer sub-scale x small
integer quant or codebook value, and the 0.5/0.25 factors of the IQ2/IQ3 types) is exact in
double precision, so the values returned here equal the reference's to the last bit.
"""
from __future__ import annotations

import numpy as np

# GGUF type ids (engine/csrc/common/qwen_quant.cuh:17-33)
F32, F16, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 0, 1, 8, 10, 11, 12, 13, 14
IQ2_XXS, IQ2_XS, IQ3_XXS, IQ4_NL, IQ3_S, IQ2_S, IQ4_XS = 16, 17, 18, 20, 21, 22, 23

# type -> (weights per block, bytes per block)  (engine/csrc/common/qwen_quant.cuh:40-58)
TRAITS = {
    F32: (1, 4), F16: (1, 2), Q8_0: (32, 34), Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144),
    Q5_K: (256, 176), Q6_K: (256, 210), IQ4_NL: (32, 18), IQ3_S: (256, 110), IQ4_XS: (256, 136),
    IQ2_XXS: (256, 66), IQ2_XS: (256, 74), IQ2_S: (256, 82), IQ3_XXS: (256, 98),
}

# The 16 non-linear 4-bit levels of IQ4_NL / IQ4_XS (engine/src/vinf/gguf/dequant.py:298).
IQ4_NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float64)


def ksigns_iq2xs() -> np.ndarray:
    """The 128-entry sign table of IQ2_XXS / IQ2_XS / IQ3_XXS: entry i is i with bit 7 set so
    that the byte has even parity.  (Checked against the reference's table in the golden test.)"""
    i = np.arange(128, dtype=np.uint8)
    parity = np.zeros(128, dtype=np.uint8)
    for b in range(7):
        parity ^= (i >> b) & 1
    return i | (parity << 7)


def _f16(blk: np.ndarray, off: int) -> np.ndarray:
    return np.ascontiguousarray(blk[:, off : off + 2]).view("<f2").astype(np.float64)[:, 0]


def _u32(blk: np.ndarray, off: int, count: int = 1) -> np.ndarray:
    return np.ascontiguousarray(blk[:, off : off + 4 * count]).view("<u4").astype(np.int64)


def _signs(bits: np.ndarray, width: int = 8, first: int = 0) -> np.ndarray:
    """bits[...] -> [..., width] of +1.0 / -1.0 (bit set = negative), dequant.py:431-435."""
    j = np.arange(first, first + width)
    return np.where((bits[..., None].astype(np.int64) >> j) & 1, -1.0, 1.0)


def _k4_scale_min(s: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """12 packed bytes -> 8 six-bit scales and 8 six-bit mins (dequant.py:205-211)."""
    s = s.astype(np.int64)
    sc = np.empty((s.shape[0], 8), dtype=np.int64)
    mn = np.empty((s.shape[0], 8), dtype=np.int64)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def _q8_0(blk, cb):  # dequant.py:283-295
    return _f16(blk, 0)[:, None] * blk[:, 2:34].view(np.int8).astype(np.float64)


def _iq4_nl(blk, cb):  # dequant.py:301-315
    qs = blk[:, 2:18]
    q = np.concatenate([qs & 0x0F, qs >> 4], axis=1)
    return _f16(blk, 0)[:, None] * IQ4_NL_VALUES[q]


def _q4_k(blk, cb):  # dequant.py:176-202
    d, dmin = _f16(blk, 0), _f16(blk, 2)
    sc, mn = _k4_scale_min(blk[:, 4:16])
    qs = blk[:, 16:144].reshape(-1, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float64)
    dl = (d[:, None] * sc)[:, :, None]
    ml = (dmin[:, None] * mn)[:, :, None]
    return (dl * q - ml).reshape(-1, 256)


def _q5_k(blk, cb):  # dequant.py:214-251
    d, dmin = _f16(blk, 0), _f16(blk, 2)
    sc, mn = _k4_scale_min(blk[:, 4:16])
    qh = blk[:, 16:48].astype(np.int64)
    qs = blk[:, 48:176].reshape(-1, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.int64)
    hi = (qh[:, None, :] >> np.arange(8)[None, :, None]) & 1
    q = (q + 16 * hi).astype(np.float64)
    dl = (d[:, None] * sc)[:, :, None]
    ml = (dmin[:, None] * mn)[:, :, None]
    return (dl * q - ml).reshape(-1, 256)


def _q6_k(blk, cb):  # dequant.py:254-280
    ql = blk[:, 0:128].reshape(-1, 2, 2, 32).astype(np.int64)  # [chunk][half][idx]
    qh = blk[:, 128:192].reshape(-1, 2, 32).astype(np.int64)  # [chunk][idx]
    scales = blk[:, 192:208].view(np.int8).astype(np.float64)
    d = _f16(blk, 208)
    out = np.empty((blk.shape[0], 2, 4, 32), dtype=np.int64)  # [chunk][quarter][idx]
    for quarter in range(4):
        half, shift = quarter % 2, 4 * (quarter // 2)
        low = (ql[:, :, half, :] >> shift) & 0x0F
        high = (qh >> (2 * quarter)) & 0x03
        out[:, :, quarter, :] = (low | (high << 4)) - 32
    q = out.reshape(-1, 16, 16).astype(np.float64)
    return ((d[:, None] * scales)[:, :, None] * q).reshape(-1, 256)


def _q2_k(blk, cb):  # dequant.py:121-139
    sc = blk[:, 0:16].astype(np.int64)
    qs = blk[:, 16:80].reshape(-1, 2, 32).astype(np.int64)
    d, dmin = _f16(blk, 80), _f16(blk, 82)
    q = np.stack([(qs >> (2 * j)) & 3 for j in range(4)], axis=2)  # [half][j][idx]
    q = q.reshape(-1, 16, 16).astype(np.float64)
    dl = (d[:, None] * (sc & 0x0F))[:, :, None]
    ml = (dmin[:, None] * (sc >> 4))[:, :, None]
    return (dl * q - ml).reshape(-1, 256)


def _q3_k(blk, cb):  # dequant.py:142-173
    hm = blk[:, 0:32].astype(np.int64)
    qs = blk[:, 32:96].reshape(-1, 2, 32).astype(np.int64)
    s = blk[:, 96:108].astype(np.int64)
    d = _f16(blk, 108)
    k = np.arange(16)
    low = (s[:, k % 8] >> (4 * (k // 8))) & 0x0F
    high = (s[:, 8 + k % 4] >> (2 * (k // 4))) & 0x03
    scales = ((low | (high << 4)) - 32).astype(np.float64)
    lowq = np.stack([(qs >> (2 * j)) & 3 for j in range(4)], axis=2).reshape(-1, 8, 32)  # [e // 32][e % 32]
    hbit = (hm[:, None, :] >> np.arange(8)[None, :, None]) & 1
    q = (lowq - np.where(hbit, 0, 4)).reshape(-1, 16, 16).astype(np.float64)
    return ((d[:, None] * scales)[:, :, None] * q).reshape(-1, 256)


def _iq4_xs(blk, cb):  # dequant.py:318-343
    d = _f16(blk, 0)
    scales_h = np.ascontiguousarray(blk[:, 2:4]).view("<u2").astype(np.int64)[:, 0]
    scales_l = blk[:, 4:8].astype(np.int64)
    g = np.arange(8)
    low = (scales_l[:, g // 2] >> (4 * (g % 2))) & 0x0F
    high = (scales_h[:, None] >> (2 * g)) & 0x03
    ls = ((low | (high << 4)) - 32).astype(np.float64)
    qs = blk[:, 8:136].reshape(-1, 8, 16)
    q = np.concatenate([qs & 0x0F, qs >> 4], axis=2)
    return ((d[:, None] * ls)[:, :, None] * IQ4_NL_VALUES[q]).reshape(-1, 256)


def _iq3_s(blk, cb):  # dequant.py:346-369
    grid = np.frombuffer(cb["iq3s_grid"], dtype=np.uint8).reshape(512, 4).astype(np.float64)
    d = _f16(blk, 0)
    qs = blk[:, 2:66].astype(np.int64)
    qh = blk[:, 66:74].astype(np.int64)
    signs = blk[:, 74:106]
    scales = blk[:, 106:110].astype(np.int64)
    idx = np.arange(64)
    entry = qs | (((qh[:, idx // 8] >> (idx % 8)) & 1) << 8)
    mag = grid[entry].reshape(-1, 256)
    g = np.arange(8)
    nib = (scales[:, g // 2] >> (4 * (g % 2))) & 0x0F
    db = d[:, None] * (1 + 2 * nib).astype(np.float64)
    sg = _signs(signs).reshape(-1, 256)
    return (db[:, :, None] * (mag * sg).reshape(-1, 8, 32)).reshape(-1, 256)


def _iq2_xxs(blk, cb):  # dequant.py:438-451
    grid = np.frombuffer(cb["iq2xxs_grid"], dtype=np.uint8).reshape(256, 8).astype(np.float64)
    ks = ksigns_iq2xs()
    d = _f16(blk, 0)
    aux = _u32(blk, 2, 16).reshape(-1, 8, 2)
    aux0, aux1 = aux[:, :, 0], aux[:, :, 1]
    db = d[:, None] * (0.5 + (aux1 >> 28).astype(np.float64)) * 0.25
    l = np.arange(4)
    entry = (aux0[:, :, None] >> (8 * l)) & 0xFF
    sbits = ks[(aux1[:, :, None] >> (7 * l)) & 127]
    vals = grid[entry] * _signs(sbits)  # [blk][ib32][l][8]
    return (db[:, :, None, None] * vals).reshape(-1, 256)


def _iq2_xs(blk, cb):  # dequant.py:454-467
    grid = np.frombuffer(cb["iq2xs_grid"], dtype=np.uint8).reshape(512, 8).astype(np.float64)
    ks = ksigns_iq2xs()
    d = _f16(blk, 0)
    q = np.ascontiguousarray(blk[:, 2:66]).view("<u2").astype(np.int64).reshape(-1, 8, 4)
    sc = blk[:, 66:74].astype(np.int64)
    nib = np.stack([sc & 0x0F, sc & 0x0F, sc >> 4, sc >> 4], axis=2)  # db[l // 2]
    db = d[:, None, None] * (0.5 + nib.astype(np.float64)) * 0.25
    vals = grid[q & 511] * _signs(ks[q >> 9])
    return (db[:, :, :, None] * vals).reshape(-1, 256)


def _iq2_s(blk, cb):  # dequant.py:470-483
    grid = np.frombuffer(cb["iq2s_grid"], dtype=np.uint8).reshape(1024, 8).astype(np.float64)
    d = _f16(blk, 0)
    qs = blk[:, 2:34].astype(np.int64).reshape(-1, 8, 4)
    sg = blk[:, 34:66].reshape(-1, 8, 4)
    qh = blk[:, 66:74].astype(np.int64)
    sc = blk[:, 74:82].astype(np.int64)
    l = np.arange(4)
    entry = qs | ((qh[:, :, None] << (8 - 2 * l)) & 0x300)
    nib = np.stack([sc & 0x0F, sc & 0x0F, sc >> 4, sc >> 4], axis=2)
    db = d[:, None, None] * (0.5 + nib.astype(np.float64)) * 0.25
    vals = grid[entry] * _signs(sg)
    return (db[:, :, :, None] * vals).reshape(-1, 256)


def _iq3_xxs(blk, cb):  # dequant.py:486-500
    grid = np.frombuffer(cb["iq3xxs_grid"], dtype=np.uint8).reshape(256, 4).astype(np.float64)
    ks = ksigns_iq2xs()
    d = _f16(blk, 0)
    qs = blk[:, 2:66].astype(np.int64).reshape(-1, 8, 4, 2)
    aux = _u32(blk, 66, 8)
    db = d[:, None] * (0.5 + (aux >> 28).astype(np.float64)) * 0.5
    l = np.arange(4)
    sbits = ks[(aux[:, :, None] >> (7 * l)) & 127]  # [blk][ib32][l]
    sg = _signs(sbits).reshape(-1, 8, 4, 2, 4)  # bits 0-3 -> first entry, 4-7 -> second
    vals = grid[qs] * sg
    return (db[:, :, None, None, None] * vals).reshape(-1, 256)


_DEQUANT = {
    Q8_0: _q8_0, IQ4_NL: _iq4_nl, Q4_K: _q4_k, Q5_K: _q5_k, Q6_K: _q6_k, Q2_K: _q2_k, Q3_K: _q3_k,
    IQ4_XS: _iq4_xs, IQ3_S: _iq3_s, IQ2_XXS: _iq2_xxs, IQ2_XS: _iq2_xs, IQ2_S: _iq2_s, IQ3_XXS: _iq3_xxs,
}


def dequantize(raw, tensor_type: int, numel: int, codebooks: dict[str, bytes] | None = None) -> np.ndarray:
    """Raw GGUF bytes -> float64 values, one per weight (dequant.py:17-57)."""
    tensor_type = int(tensor_type)
    if tensor_type not in TRAITS:
        raise ValueError(f"no dequantiser for GGUF type {tensor_type}")
    block, size = TRAITS[tensor_type]
    data = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.reshape(-1).view(np.uint8)
    if numel % block or data.size != numel // block * size:
        raise ValueError("tensor data length does not match the tensor shape")
    if tensor_type == F32:
        return data.view("<f4").astype(np.float64)
    if tensor_type == F16:
        return data.view("<f2").astype(np.float64)
    return _DEQUANT[tensor_type](data.reshape(-1, size), codebooks or {}).reshape(-1)


def matvec(raw, tensor_type: int, rows: int, cols: int, x: np.ndarray,
           codebooks: dict[str, bytes] | None = None, chunk_rows: int = 2048) -> np.ndarray:
    """y[t][r] = sum_k W[r][k] * x[t][k] in double precision; x is [ntok, cols] (or [cols]).
    This is dequantise + matvec_reference (engine/tests/test_phase30_cuda_qmatvec.py:60-63)."""
    x2 = np.atleast_2d(np.asarray(x, dtype=np.float64))
    block, size = TRAITS[int(tensor_type)]
    rb = cols // block * size
    data = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.reshape(-1).view(np.uint8)
    out = np.empty((x2.shape[0], rows), dtype=np.float64)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        w = dequantize(data[r0 * rb : r1 * rb], tensor_type, (r1 - r0) * cols, codebooks).reshape(r1 - r0, cols)
        out[:, r0:r1] = x2 @ w.T
    return out if np.ndim(x) == 2 else out[0]


def argmax_rows(logits: np.ndarray) -> np.ndarray:
    """Row-wise argmax, lowest index on ties; a row with no value above -inf gives 0x7fffffff
    (engine/csrc/megakernel/qwen_runtime.cu:851-876)."""
    logits = np.atleast_2d(logits)
    out = np.empty(logits.shape[0], dtype=np.int64)
    for t, row in enumerate(logits):
        best, idx = -np.inf, 0x7FFFFFFF
        valid = row > -np.inf  # NaN compares false, like the kernel's strict '>'
        if valid.any():
            masked = np.where(valid, row, -np.inf)
            best = masked.max()
            idx = int(np.flatnonzero(masked == best)[0])
        out[t] = idx
    return out


def cpu_qwen_bound(raw, tensor_type: int, rows: int, cols: int, x: np.ndarray,
                   codebooks: dict[str, bytes] | None = None) -> np.ndarray:
    """Per-output error allowance of the reference CPU path, whose activations are rounded to int8
    per 32 elements: 1.05 * sum_g(sum_i |w_i| * amax_g / 254) (engine/tests/test_phase31e_cpu_layers.py:44-51)."""
    x2 = np.atleast_2d(np.asarray(x, dtype=np.float64))
    w = np.abs(dequantize(raw, tensor_type, rows * cols, codebooks)).reshape(rows, cols // 32, 32).sum(axis=2)
    amax = np.abs(x2).reshape(x2.shape[0], cols // 32, 32).max(axis=2)
    return 1.05 * (amax / 254.0) @ w.T


def fused_matvec(raw, tensor_type: int, rows: int, cols: int, x, codebooks=None, *, x2=None, norm_w=None, eps: float = 1e-6, residual=None):
    """y = W v (+ residual) in double precision with the activation prologues of the reference's fused QMV instruction
    (engine/csrc/megakernel/qwen_megakernel.cu:486-550): v = silu(x) * x2 if x2 is given, else x; with norm_w,
    v * rsqrt(mean(v^2) + eps) * norm_w per activation row; `:231`: the result is added to what y held.  Test infrastructure."""
    v = np.atleast_2d(np.asarray(x, dtype=np.float64))
    if x2 is not None:
        v = v / (1.0 + np.exp(-v)) * np.atleast_2d(np.asarray(x2, dtype=np.float64))
    if norm_w is not None:
        v = v / np.sqrt(np.mean(v * v, axis=1, keepdims=True) + eps) * np.asarray(norm_w, dtype=np.float64)[None, :]
    w = dequantize(raw, tensor_type, rows * cols, codebooks).reshape(rows, cols)
    y = v @ w.T
    return y if residual is None else y + np.asarray(residual, dtype=np.float64)
