"""Regenerates the golden fixtures in this directory from the reference implementation.

Run in a container that has the reference checkout (it cannot run on the GPU box):

    python tests/golden/make_golden.py /path/to/reference/engine

Writes
  iq_codebooks.npz     the IQ codebooks the reference keeps as data
                       (engine/src/vinf/gguf/iq_tables.py:347, engine/src/vinf/cuda/qwen_runtime.py:41-44)
  dequant_golden.npz   for each of the 15 matvec types: seeded random blocks in the recipe of
                       engine/tests/test_phase30_cuda_qmatvec.py:45-57 and the values the reference
                       dequantiser (engine/src/vinf/gguf/dequant.py:17-57) returns for them
  cpu_qwen_golden.npz  outputs of the reference CPU matvec (engine/csrc/cpu/qwen_cpu.c:581-641) on the
                       shapes of engine/tests/test_phase31e_cpu_layers.py:53-60, if oracle/_ref holds a
                       build of it (make -C oracle ref)
"""
from __future__ import annotations

import importlib.util
import random
import struct
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
if len(sys.argv) != 2:
    sys.exit(__doc__)
ENGINE = Path(sys.argv[1])
sys.path.insert(0, str(ENGINE / "src"))
sys.path.insert(0, str(REPO))

from vinf.cuda.qwen_runtime import _iq3_s_grid_bytes  # noqa: E402
from vinf.gguf.dequant import dequantize_tensor  # noqa: E402
from vinf.gguf.iq_tables import iq_table  # noqa: E402
from vinf.gguf.parser import GGUFTensorInfo, GGUFTensorType  # noqa: E402

from vinf_3080ti_b200.gguf_types import F16_FIELDS, TRAITS  # noqa: E402

TYPES = sorted(TRAITS)


def synthetic_rows(tensor_type, rows: int, cols: int, rng: random.Random) -> bytes:
    block, size = TRAITS[tensor_type]
    if tensor_type.name == "F32":
        return struct.pack(f"<{rows * cols}f", *(rng.uniform(-1, 1) for _ in range(rows * cols)))
    if tensor_type.name == "F16":
        return struct.pack(f"<{rows * cols}e", *(rng.uniform(-1, 1) for _ in range(rows * cols)))
    out = bytearray()
    for _ in range(rows * cols // block):
        blk = bytearray(rng.getrandbits(8) for _ in range(size))
        for off in F16_FIELDS[tensor_type]:
            blk[off : off + 2] = struct.pack("<e", rng.uniform(0.001, 0.05))
        out.extend(blk)
    return bytes(out)


def main() -> None:
    books = {name: np.frombuffer(iq_table(name), dtype=np.uint8)
             for name in ("iq2xxs_grid", "iq2xs_grid", "iq2s_grid", "iq3xxs_grid", "ksigns_iq2xs")}
    books["iq3s_grid"] = np.frombuffer(_iq3_s_grid_bytes(), dtype=np.uint8)
    np.savez_compressed(HERE / "iq_codebooks.npz", **books)

    rng = random.Random(30)
    rows, cols = 5, 512
    golden = {}
    for t in TYPES:
        raw = synthetic_rows(t, rows, cols, rng)
        info = GGUFTensorInfo("w", (rows * cols,), GGUFTensorType(int(t)), 0, 0)
        values = np.array(dequantize_tensor(info, memoryview(raw)).values, dtype=np.float64)
        assert np.array_equal(values.astype(np.float32).astype(np.float64), values), t  # fp32-representable
        golden[f"raw_{int(t)}"] = np.frombuffer(raw, dtype=np.uint8)
        golden[f"val_{int(t)}"] = values.astype(np.float32)
    golden["shape"] = np.array([rows, cols])
    np.savez_compressed(HERE / "dequant_golden.npz", **golden)

    ref = sorted((REPO / "oracle" / "_ref").glob("_cpu_qwen*.so"))
    if not ref:
        print("oracle/_ref/_cpu_qwen*.so not built: cpu_qwen_golden.npz left as it is")
        return
    spec = importlib.util.spec_from_file_location("_cpu_qwen", ref[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rt = mod.CpuRuntime(bytes(books["iq3s_grid"]), 4)
    rng = random.Random(3101)
    rows, cols, ntok = 12, 512, 3
    out = {"shape": np.array([rows, cols, ntok])}
    keep = []
    for t in TYPES:
        raw = synthetic_rows(t, rows, cols, rng)
        x = np.array([[rng.uniform(-1, 1) for _ in range(cols)] for _ in range(ntok)], dtype=np.float32)
        name = f"w{int(t)}"
        keep.append(raw)
        rt.add_tensor(name, raw, int(t), cols, rows)
        rt.alloc(name + ".x", cols * ntok)
        rt.alloc(name + ".y", rows * ntok)
        rt.write(name + ".x", x.tobytes())
        rt.qmv(name, name + ".x", name + ".y", ntok)
        out[f"raw_{int(t)}"] = np.frombuffer(raw, dtype=np.uint8)
        out[f"x_{int(t)}"] = x
        out[f"y_{int(t)}"] = np.frombuffer(rt.read(name + ".y"), dtype=np.float32).reshape(ntok, rows).copy()
    np.savez_compressed(HERE / "cpu_qwen_golden.npz", **out)


if __name__ == "__main__":
    main()
