"""Host-side mirror of the reference's device runtime for the quantized-matvec path.

`Runtime` has the method names, argument orders, defaults and exception types of the reference's CPython
type `vinf._cuda_qwen_runtime.Runtime` (engine/csrc/megakernel/qwen_runtime.cu:2602-2704) for everything on
the matvec path, so an executor that is handed one as its `runtime=` (engine/src/vinf/qwen_gpu.py:227,253-259)
calls it unchanged.  The reference's thin Python wrapper (engine/src/vinf/cuda/qwen_runtime.py:47-116) keeps working
on top of it: it only forwards to whatever module object its loader returns.

All work is done by libvinf_b200.so through its C ABI; this file only converts arguments and errors.
Weights are always resident in HBM, so the reference's host-staging / VMM-group methods are kept as
no-ops with trivial answers.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np

from . import _capi
from .gguf_types import CODEBOOK_BYTES

MAX_ARGMAX_ROWS = 256  # engine/csrc/megakernel/qwen_runtime.cu:573


def _ptr(data) -> tuple[np.ndarray, int, int]:
    """Any bytes-like object -> (keep-alive array, address, byte length), without copying."""
    arr = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1).view(np.uint8)
    if not arr.flags.c_contiguous:
        arr = np.ascontiguousarray(arr)
    return arr, arr.ctypes.data, arr.size


def _name(s: str | None):
    return None if s is None else s.encode("utf-8")


def reference_codebooks() -> dict[str, bytes]:
    """The IQ codebooks, taken from an importable `vinf` (the reference keeps them as data in
    engine/src/vinf/gguf/iq_tables.py:347 and engine/src/vinf/cuda/qwen_runtime.py:41-44).  Empty when
    `vinf` is not importable; a caller can then pass `codebooks=` itself."""
    try:
        from vinf.cuda.qwen_runtime import _iq3_s_grid_bytes
        from vinf.gguf.iq_tables import iq_table
    except ImportError:
        return {}
    books = {name: iq_table(name) for name in ("iq2xxs_grid", "iq2xs_grid", "iq2s_grid", "iq3xxs_grid")}
    books["iq3s_grid"] = _iq3_s_grid_bytes()
    return books


PROBE_KINDS = ("PRMT", "LOP3", "FFMA2", "FFMA", "IMAD", "SHF", "cvt.f32.f16", "PRMT+FFMA2 alternating",
               "decode of 8 Q4_K weights, 1 activation row", "decode of 8 Q4_K weights, 4 activation rows")


def probe_issue_rates(warps_per_sm: int = 16) -> dict[str, float]:
    """Scheduler cycles per warp instruction (last two entries: per 8 weights of a row) on the current device, measured by
    the library's probe kernel.  What the instruction-issue roofline of the matvec kernels is built on."""
    lib = _capi.load()
    out = (ctypes.c_double * len(PROBE_KINDS))()
    _capi.check(lib.vqm_probe_issue_rates(int(warps_per_sm), out, len(PROBE_KINDS)))
    return dict(zip(PROBE_KINDS, (float(v) for v in out)))


class Runtime:
    """Named raw-GGUF weight tensors and fp32 buffers in B200 HBM, with y = W x and argmax on them."""

    def __init__(self, iq3s_grid: bytes | None = None, codebooks: dict[str, bytes] | None = None) -> None:
        self._lib = _capi.load()
        self._h = ctypes.c_void_p()
        if iq3s_grid is not None and len(iq3s_grid) != 2048:
            raise ValueError("iq3s_grid must be 2048 bytes (512 entries x 4 values)")
        keep, addr, n = _ptr(iq3s_grid) if iq3s_grid is not None else (None, None, 0)
        _capi.check(self._lib.vqm_runtime_create(addr, n, ctypes.byref(self._h)))
        for name, data in (codebooks or {}).items():
            if name in CODEBOOK_BYTES:
                self.set_codebook(name, data)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.vqm_runtime_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self) -> None:  # tp_dealloc: engine/csrc/megakernel/qwen_runtime.cu:1299-1336
        try:
            self.close()
        except Exception:
            pass

    # ---- codebooks ---------------------------------------------------------------------------------
    def set_codebook(self, name: str, data: bytes) -> None:
        keep, addr, n = _ptr(data)
        _capi.check(self._lib.vqm_set_codebook(self._h, _name(name), addr, n))

    # ---- weights -----------------------------------------------------------------------------------
    def upload(self, name: str, data, type: int, cols: int, rows: int, resident: bool = True, group: int = -1) -> None:
        """upload(name, raw_bytes, gguf_type_id, cols, rows[, resident, group]); resident/group are
        accepted and ignored (everything is resident)."""
        keep, addr, n = _ptr(data)
        _capi.check(self._lib.vqm_upload(self._h, _name(name), addr, n, int(type), int(cols), int(rows)))

    def upload_file(self, name: str, path, offset: int, nbytes: int, type: int, cols: int, rows: int, threads: int = 4) -> None:
        """The tensor's raw blocks straight from `nbytes` bytes at byte `offset` of the file `path` (for a GGUF file the
        tensor's absolute offset): parallel reads into pinned staging overlapped with the copies to the device.  Replaces the
        reference wrapper's mmap + upload per tensor (engine/src/vinf/cuda/qwen_runtime.py:68-86)."""
        if offset < 0 or nbytes < 0:
            raise ValueError("offset and nbytes must be non-negative")
        _capi.check(self._lib.vqm_upload_file(self._h, _name(name), _name(str(path)), int(offset), int(nbytes), int(type), int(cols), int(rows),
                                              int(threads)))

    def bind_tensor(self, name: str, device_ptr: int, type: int, cols: int, rows: int) -> None:
        """Registers raw blocks that already sit in device memory (not freed by the runtime)."""
        _capi.check(self._lib.vqm_bind_tensor(self._h, _name(name), ctypes.c_void_p(device_ptr), int(type), int(cols), int(rows)))

    def free(self, name: str) -> None:
        _capi.check(self._lib.vqm_free(self._h, _name(name)))

    def has(self, name: str) -> bool:
        out = ctypes.c_int()
        _capi.check(self._lib.vqm_has(self._h, _name(name), ctypes.byref(out)))
        return bool(out.value)

    def device_bytes(self) -> int:
        out = ctypes.c_size_t()
        _capi.check(self._lib.vqm_device_bytes(self._h, ctypes.byref(out)))
        return out.value

    def tensor_info(self, name: str) -> tuple[int, int, int, int, int, int, bool]:
        info = _capi.TensorInfo()
        _capi.check(self._lib.vqm_tensor_info(self._h, _name(name), ctypes.byref(info)))
        return (info.addr, info.type, info.rows, info.cols, info.row_bytes, info.nbytes, bool(info.resident))

    # ---- buffers -----------------------------------------------------------------------------------
    def alloc(self, name: str, n: int, elem: int = 4, virtual: bool = False) -> None:
        if n <= 0:
            raise ValueError(f"buffer {name} size must be positive")
        _capi.check(self._lib.vqm_alloc(self._h, _name(name), int(n), int(elem)))

    def bind(self, name: str, device_ptr: int, n: int, elem: int = 4) -> None:
        """Registers caller-owned device memory (for instance a torch tensor's) under a buffer name."""
        _capi.check(self._lib.vqm_bind(self._h, _name(name), ctypes.c_void_p(device_ptr), int(n), int(elem)))

    def release(self, name: str) -> None:
        _capi.check(self._lib.vqm_release(self._h, _name(name)))

    def write(self, name: str, data, offset: int = 0) -> None:
        if offset < 0:
            raise ValueError(f"write to {name}: bad offset")
        keep, addr, n = _ptr(data)
        _capi.check(self._lib.vqm_write(self._h, _name(name), addr, n, int(offset)))

    def read(self, name: str, n: int = -1, offset: int = 0) -> bytes:
        if offset < 0:
            raise ValueError("bad read offset")
        elem = self.buffer_elem(name)
        if n < 0:
            total = self._buffer_len(name)
            if offset > total:
                raise ValueError("bad read offset")
            n = total - offset
        out = np.empty(n * elem, dtype=np.uint8)
        _capi.check(self._lib.vqm_read(self._h, _name(name), out.ctypes.data, int(n), int(offset)))
        return out.tobytes()

    def read_array(self, name: str, n: int = -1, offset: int = 0) -> np.ndarray:
        """read() as a float32 / float16 numpy array (no reference counterpart; saves a copy)."""
        data = self.read(name, n, offset)
        return np.frombuffer(data, dtype=np.float32 if self.buffer_elem(name) == 4 else np.float16)

    def copy(self, dst: str, dst_off: int, src: str, src_off: int, n: int) -> None:
        if dst_off < 0 or src_off < 0 or n < 0:
            raise ValueError("offsets and count must be non-negative")
        _capi.check(self._lib.vqm_copy(self._h, _name(dst), int(dst_off), _name(src), int(src_off), int(n)))

    def zero(self, name: str) -> None:
        _capi.check(self._lib.vqm_zero(self._h, _name(name)))

    def zero_range(self, name: str, offset: int, n: int) -> None:
        if offset < 0 or n < 0:
            raise ValueError("zero_range out of bounds")
        _capi.check(self._lib.vqm_zero_range(self._h, _name(name), int(offset), int(n)))

    def buffer_ptr(self, name: str) -> tuple[int, int]:
        addr, n = ctypes.c_uint64(), ctypes.c_size_t()
        _capi.check(self._lib.vqm_buffer_ptr(self._h, _name(name), ctypes.byref(addr), ctypes.byref(n)))
        return addr.value, n.value

    def buffer_elem(self, name: str) -> int:
        out = ctypes.c_int()
        _capi.check(self._lib.vqm_buffer_elem(self._h, _name(name), ctypes.byref(out)))
        return out.value

    def _buffer_len(self, name: str) -> int:
        out = ctypes.c_size_t()
        _capi.check(self._lib.vqm_buffer_len(self._h, _name(name), ctypes.byref(out)))
        return out.value

    def buffer_bytes(self) -> int:
        out = ctypes.c_size_t()
        _capi.check(self._lib.vqm_buffer_bytes(self._h, ctypes.byref(out)))
        return out.value

    # ---- the hot path --------------------------------------------------------------------------------
    def qmv(self, weight: str, x: str, y: str, ntok: int = 1) -> None:
        """y[t][r] = sum_k W[r][k] x[t][k]; asynchronous."""
        _capi.check(self._lib.vqm_qmv(self._h, _name(weight), _name(x), _name(y), int(ntok)))

    def matvec(self, name: str, x) -> bytes:
        """matvec(name, x_f32_bytes) -> y_f32_bytes; synchronous single-row entry."""
        keep, addr, n = _ptr(x)
        if not self.has(name):
            raise KeyError(f"{name} is not resident on the GPU")
        rows = self.tensor_info(name)[2]
        out = np.empty(rows, dtype=np.float32)
        _capi.check(self._lib.vqm_matvec(self._h, _name(name), addr, n, out.ctypes.data, out.nbytes))
        return out.tobytes()

    def argmax(self, x: str, n: int) -> int:
        out = ctypes.c_int()
        _capi.check(self._lib.vqm_argmax(self._h, _name(x), int(n), ctypes.byref(out)))
        return out.value

    def argmax_rows(self, x: str, n: int, ntok: int) -> list[int]:
        if ntok < 1 or ntok > MAX_ARGMAX_ROWS:
            raise ValueError(f"ntok must be in [1, {MAX_ARGMAX_ROWS}]")
        out = (ctypes.c_int * ntok)()
        _capi.check(self._lib.vqm_argmax_rows(self._h, _name(x), int(n), int(ntok), out))
        return list(out)

    def qmv_argmax(self, weight: str, x: str, y: str | None, ntok: int = 1, blocking: bool = True) -> list[int] | None:
        """The LM head in one launch: qmv(weight, x, y, ntok) then argmax_rows(y, rows, ntok).
        y=None skips storing the logits.  blocking=False leaves the ids on the device (argmax_result)."""
        if ntok < 1 or ntok > 8:
            raise ValueError("ntok must be in [1, 8] for the fused argmax")
        out = (ctypes.c_int * ntok)() if blocking else None
        _capi.check(self._lib.vqm_qmv_argmax(self._h, _name(weight), _name(x), _name(y), int(ntok), out))
        return list(out) if blocking else None

    def qmv_fused(self, weight: str, x: str, y: str | None, ntok: int = 1, *, add: bool = False, norm: str | None = None, eps: float = 1e-6,
                  silu_mul: str | None = None, argmax: bool = False, blocking: bool = True) -> list[int] | None:
        """qmv with the reference's fused-QMV prologues and epilogues (engine/csrc/common/qwen_mk_abi.h:55-58): the activations
        are silu(x) * silu_mul if `silu_mul` names a second buffer, then rms-normalised and scaled by the weights `norm`
        (a buffer or F32 tensor of `cols` values) if given; `add` makes it y += W v; `argmax` adds the fused argmax and
        returns the ids (blocking) or leaves them on the device."""
        flags = (1 if add else 0) | (2 if norm is not None else 0) | (4 if argmax else 0) | (8 if silu_mul is not None else 0)
        out = (ctypes.c_int * ntok)() if (argmax and blocking) else None
        _capi.check(self._lib.vqm_qmv_fused(self._h, _name(weight), _name(x), _name(y), int(ntok), flags, _name(silu_mul), _name(norm), float(eps), out))
        return list(out) if out is not None else None

    def argmax_result(self) -> tuple[int, int]:
        """Device addresses of the last fused argmax: (int32 ids[8], fp32 values[8])."""
        ids, vals = ctypes.c_uint64(), ctypes.c_uint64()
        _capi.check(self._lib.vqm_argmax_result(self._h, ctypes.byref(ids), ctypes.byref(vals)))
        return ids.value, vals.value

    def argmax_fetch(self, ntok: int, with_values: bool = False):
        """Blocking read of the last fused argmax: ids, or (ids, values)."""
        ids = (ctypes.c_int * ntok)()
        vals = (ctypes.c_float * ntok)() if with_values else None
        _capi.check(self._lib.vqm_argmax_fetch(self._h, int(ntok), ids, vals))
        return (list(ids), list(vals)) if with_values else list(ids)

    def set_argmax_row_base(self, weight: str, row_base: int) -> None:
        _capi.check(self._lib.vqm_set_argmax_row_base(self._h, _name(weight), int(row_base)))

    def dequantize(self, weight: str, out: str) -> None:
        """Exact fp32 values of a weight tensor into an fp32 buffer (rows * cols elements)."""
        _capi.check(self._lib.vqm_dequantize(self._h, _name(weight), _name(out)))

    def set_gemm_min_rows(self, n: int) -> None:
        _capi.check(self._lib.vqm_set_gemm_min_rows(self._h, int(n)))

    def synchronize(self) -> None:
        _capi.check(self._lib.vqm_synchronize(self._h))

    def mem_info(self) -> tuple[int, int]:
        free, total = ctypes.c_size_t(), ctypes.c_size_t()
        _capi.check(self._lib.vqm_mem_info(ctypes.byref(free), ctypes.byref(total)))
        return free.value, total.value

    # ---- stream / graphs (no reference counterpart) --------------------------------------------------
    def stream(self) -> int:
        """The runtime's cudaStream_t as an integer (wrap with torch.cuda.ExternalStream to time on it)."""
        return int(self._lib.vqm_stream(self._h) or 0)

    def set_stream(self, stream: int | None) -> None:
        """Launch on a caller-owned cudaStream_t (None: back to the runtime's own stream)."""
        _capi.check(self._lib.vqm_set_stream(self._h, ctypes.c_void_p(stream) if stream else None))

    def capture_begin(self) -> None:
        _capi.check(self._lib.vqm_capture_begin(self._h))

    def capture_end(self) -> int:
        out = ctypes.c_int()
        _capi.check(self._lib.vqm_capture_end(self._h, ctypes.byref(out)))
        return out.value

    def graph_launch(self, graph_id: int) -> None:
        _capi.check(self._lib.vqm_graph_launch(self._h, int(graph_id)))

    def graph_destroy(self, graph_id: int) -> None:
        _capi.check(self._lib.vqm_graph_destroy(self._h, int(graph_id)))

    def launch_count(self) -> int:
        out = ctypes.c_uint64()
        _capi.check(self._lib.vqm_launch_count(self._h, ctypes.byref(out)))
        return out.value

    # ---- row-sharded tensors over several GPUs (no reference counterpart) -----------------------------------------
    def exchange_create(self, nbytes: int) -> tuple[bytes, int]:
        """Allocates this rank's exchange region; returns (64-byte CUDA IPC handle, device address)."""
        handle = ctypes.create_string_buffer(64)
        addr = ctypes.c_uint64()
        _capi.check(self._lib.vqm_exchange_create(self._h, int(nbytes), handle, ctypes.byref(addr)))
        return handle.raw, addr.value

    def exchange_open(self, handle: bytes) -> int:
        """Maps a peer's exchange region from its IPC handle; returns its address in this process."""
        addr = ctypes.c_uint64()
        buf = ctypes.create_string_buffer(handle, 64)
        _capi.check(self._lib.vqm_exchange_open(self._h, buf, ctypes.byref(addr)))
        return addr.value

    def exchange_config(self, rank: int, region_addrs: Sequence[int], flag_off: int, count_off: int, n_slots: int) -> None:
        arr = (ctypes.c_uint64 * len(region_addrs))(*region_addrs)
        _capi.check(self._lib.vqm_exchange_config(self._h, len(region_addrs), int(rank), arr, int(flag_off), int(count_off), int(n_slots)))

    def qmv_push(self, weight: str, x: str, y: str, ntok: int, slot: int, dst_off: int, rows_total: int, row_begin: int,
                 wait_slot: int = -1, with_argmax: bool = False) -> None:
        """qmv on this rank's row slice fused with its all-gather (see include/vinf_b200.h)."""
        _capi.check(self._lib.vqm_qmv_push(self._h, _name(weight), _name(x), _name(y), int(ntok), int(slot), int(dst_off), int(rows_total),
                                           int(row_begin), int(wait_slot), int(with_argmax)))

    def set_column_split(self, enabled: bool) -> None:
        """Short launches share each row's columns among the blocks of a cluster (default on); off makes a tensor's
        outputs independent of what else is in its launch."""
        _capi.check(self._lib.vqm_set_column_split(self._h, int(bool(enabled))))

    def qmv_group(self, weights: list[str], x: str, ys: list[str], ntok: int) -> None:
        """ys[i] = W_i x for up to four tensors that share x, their GGUF type and their columns, in ONE launch
        (q/k/v of an attention layer, gate/up of an FFN).  No counterpart in the reference, which launches one
        kernel per tensor (engine/csrc/megakernel/qwen_runtime.cu:1259-1296)."""
        if len(weights) != len(ys):
            raise ValueError("one output buffer per tensor")
        n = len(weights)
        w = (ctypes.c_char_p * n)(*[_name(v) for v in weights])
        y = (ctypes.c_char_p * n)(*[_name(v) for v in ys])
        _capi.check(self._lib.vqm_qmv_group(self._h, n, w, _name(x), y, int(ntok)))

    def qmv_push_group(self, weights: list[str], x: str, ys: list[str], ntok: int, slot: int, dst_offs: list[int],
                       rows_totals: list[int], row_begins: list[int], wait_slot: int = -1) -> None:
        """qmv_group on this rank's row slices fused with their all-gathers: one flag slot for the launch."""
        n = len(weights)
        if not (len(ys) == len(dst_offs) == len(rows_totals) == len(row_begins) == n):
            raise ValueError("one entry per tensor")
        w = (ctypes.c_char_p * n)(*[_name(v) for v in weights])
        y = (ctypes.c_char_p * n)(*[_name(v) for v in ys])
        _capi.check(self._lib.vqm_qmv_push_group(self._h, n, w, _name(x), y, int(ntok), int(slot), (ctypes.c_size_t * n)(*dst_offs),
                                                 (ctypes.c_int * n)(*rows_totals), (ctypes.c_int * n)(*row_begins), int(wait_slot)))

    # ---- residency machinery of the reference: everything is resident here ------------------------------
    # (engine/csrc/megakernel/qwen_runtime.cu:1485-1811; engine/src/vinf/gguf/residency.py:256-354)
    def vram_bytes(self) -> int:
        return self.device_bytes() + self.buffer_bytes()

    def pinned_bytes(self) -> int:
        return 0

    def streamed_bytes(self) -> int:
        return 0

    def staging_bytes(self) -> int:
        return 0

    def set_arena(self, nbytes: int) -> None:
        return None

    def set_staging(self, nbytes: int) -> None:
        return None

    def set_stream_order(self, names, slots: int = 2) -> None:
        return None

    def reserve_ring(self, slot_bytes: int, slots: int) -> None:
        return None

    def set_weight_space(self, nbytes: int) -> None:
        return None

    def add_weight_group(self, nbytes: int) -> int:
        return -1  # "no group": upload(..., group=-1) is the plain resident path

    def demote_group(self, group: int) -> None:
        return None

    def promote_group(self, group: int) -> bool:
        return True

    def weight_groups(self) -> list:
        return []

    def map_range(self, name: str, offset: int, n: int) -> bool:
        return True

    def unmap_range(self, name: str, offset: int, n: int) -> None:
        return None

    def map_cost(self, name: str, offset: int, n: int) -> int:
        return 0

    def vmm_granularity(self) -> int:
        return 2 * 1024 * 1024
