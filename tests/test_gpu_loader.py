"""Weights from a file into HBM (Runtime.upload_file, loader.load_matrices): the device tensor must hold exactly the
file's bytes, so a matvec on it equals, bit for bit, the matvec on the same bytes uploaded from memory."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import numpy as np
import pytest

from vinf_3080ti_b200 import loader
from vinf_3080ti_b200.gguf_types import TRAITS, GGUFTensorType as T
from vinf_3080ti_b200.synth import synthetic_activations, synthetic_blocks

pytestmark = pytest.mark.gpu


@dataclass
class TensorRecord:  # the fields of the reference's GGUFTensorInfo that the loader reads
    name: str
    dimensions: tuple
    tensor_type: T
    absolute_offset: int
    nbytes: int


@dataclass
class ParsedFile:
    path: Path
    tensors: dict


@pytest.fixture(scope="module")
def rt(codebooks):
    from vinf_3080ti_b200.runtime import Runtime

    runtime = Runtime(codebooks["iq3s_grid"], codebooks)
    yield runtime
    runtime.close()


def _same_outputs(rt, a: str, b: str, rows: int, cols: int, rng) -> bool:
    x = synthetic_activations(2, cols, rng)
    rt.alloc("x", 2 * cols)
    rt.alloc("ya", 2 * rows)
    rt.alloc("yb", 2 * rows)
    rt.write("x", x)
    rt.qmv(a, "x", "ya", 2)
    rt.qmv(b, "x", "yb", 2)
    rt.synchronize()
    return np.array_equal(rt.read_array("ya").view(np.uint32), rt.read_array("yb").view(np.uint32))


@pytest.mark.parametrize("threads", [1, 3, 16])
def test_upload_file_brings_exactly_the_files_bytes(rt, tmp_path, threads):
    rng = np.random.default_rng(threads)
    rows, cols = 6000, 5120  # 25 MB of Q6_K: several 8 MiB chunks, the last one partial
    raw = synthetic_blocks(T.Q6_K, rows, cols, rng)
    path = tmp_path / "weights.bin"
    offset = 4099  # tensors of a GGUF file start at arbitrary 32-byte multiples; any offset must work
    with open(path, "wb") as f:
        f.write(bytes(offset))
        f.write(raw.tobytes())
        f.write(b"tail")
    rt.upload_file("from_file", path, offset, raw.size, int(T.Q6_K), cols, rows, threads)
    rt.upload("from_memory", raw, int(T.Q6_K), cols, rows)
    assert rt.tensor_info("from_file")[1:] == rt.tensor_info("from_memory")[1:]
    assert _same_outputs(rt, "from_file", "from_memory", rows, cols, rng)
    rt.free("from_file")
    rt.free("from_memory")


def test_upload_file_errors(rt, tmp_path):
    raw = synthetic_blocks(T.Q4_K, 4, 256, np.random.default_rng(0))
    path = tmp_path / "short.bin"
    path.write_bytes(raw.tobytes()[:-1])
    with pytest.raises(ValueError, match="bytes"):
        rt.upload_file("w", path, 0, raw.size, int(T.Q4_K), 256, 4)  # file one byte short
    with pytest.raises(ValueError, match="cannot open"):
        rt.upload_file("w", tmp_path / "missing.bin", 0, raw.size, int(T.Q4_K), 256, 4)
    with pytest.raises(ValueError):
        rt.upload_file("w", path, 0, raw.size - 1, int(T.Q4_K), 256, 4)  # byte count does not match the shape
    with pytest.raises(ValueError):
        rt.upload_file("w", path, 0, 34, 2, 32, 1)  # Q4_0: no kernel
    assert not rt.has("w")


def test_load_matrices_takes_every_matrix_of_a_parsed_file(rt, tmp_path):
    rng = np.random.default_rng(5)
    shapes = {"blk.0.attn_q.weight": (T.Q6_K, 96, 512), "blk.0.ffn_down.weight": (T.Q4_K, 64, 768), "output.weight": (T.Q8_0, 300, 256)}
    path = tmp_path / "model.gguf"
    tensors, raws = {}, {}
    with open(path, "wb") as f:
        f.write(bytes(1000))  # stands in for the header
        for name, (t, rows, cols) in shapes.items():
            pad = (-f.tell()) % 32
            f.write(bytes(pad))
            raw = synthetic_blocks(t, rows, cols, rng)
            tensors[name] = TensorRecord(name, (cols, rows), t, f.tell(), raw.size)
            raws[name] = raw
            f.write(raw.tobytes())
        norm = np.ones(512, dtype=np.float32)  # a one-dimensional tensor: not a matrix, left to the element-wise ops
        tensors["blk.0.attn_norm.weight"] = TensorRecord("blk.0.attn_norm.weight", (512,), T.F32, f.tell(), norm.nbytes)
        f.write(norm.tobytes())
    loaded = loader.load_matrices(rt, ParsedFile(path, tensors), threads=4)
    assert loaded == {name: raws[name].size for name in shapes}
    assert not rt.has("blk.0.attn_norm.weight")
    for name, (t, rows, cols) in shapes.items():
        block, size = TRAITS[t]
        assert rt.tensor_info(name)[1:4] == (int(t), rows, cols)
        rt.upload("copy", raws[name], int(t), cols, rows)
        assert _same_outputs(rt, name, "copy", rows, cols, rng)
