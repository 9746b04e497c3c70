"""Benchmark of the GGUF quantized-matvec path:  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: one decode pass over the synthetic 27B matvec set at M activation rows (default 4, the MTP k=3 verify
pass): 64 layers x {Q6_K q/k/v/o, Q3_K gate/up, Q4_K down} with hidden 5120 / FFN 17408, then the Q6_K LM head
151936 x 5120 with the fused on-device argmax - 257 launches (q/k/v and gate/up of a layer go out as one launch each)
over 12.6 GB of raw GGUF blocks, all resident in HBM.  Weights are seeded synthetic blocks (uniform-random bytes,
fp16 super-scales uniform in [1e-3, 1e-2)), activations fp32 N(0,1).  The pass is 100x larger than L2, so no flush is
needed between steps.

One JSON line on rank 0:
  metric / value   weight GB/s of the pass (weight bytes / device time), inputs resident in HBM, one CUDA graph per pass
  e2e              the same with host buffers: per step the activations are copied from pinned host memory, the pass
                   runs, the argmax ids are read back; `e2e.plugin_calls` times the call sequence the reference's
                   executor makes (write -> qmv ... -> argmax_rows, one call per launch, no graph)
  roofline         the dominant kernel (Q3_K gate/up matvec) timed alone over the model's 128 distinct tensors
  kernels          the metric's first clause: single matvec kernels at M = 1 / 4 / 8 (and the IQ sweep at M = 1 / 8), each
                   over enough distinct copies of its tensor to defeat L2
  prefill          the prompt-pass GEMM, Q4_K 17408 x 5120 with 512 activation rows
  reference_cuda_kernel   the reference's own CUDA matvec kernel (its source compiled unchanged for sm_100a) on the
                   same tensors, same GPU
  cpu_baseline     the reference's own CPU matvec on this host's cores, on the pass's byte mix
N > 1 (torchrun)   every rank owns a contiguous slice of the output rows of every tensor (strong scaling); a matvec
                   pushes its slice into every rank's gathered vector from its epilogue (default) or the slices are
                   combined with NCCL all-gathers (--gather nccl).  `multi_gpu_check` compares the pushed vectors with
                   NCCL all-gathers of the same slices and the combined argmax with the argmax of the gathered logits.
--impl reference   the reference's CPU implementation alone, on the same byte mix (64 layer sets + the LM head per step)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

from vinf_3080ti_b200.gguf_types import F16_FIELDS, TRAITS, GGUFTensorType as T  # noqa: E402
from vinf_3080ti_b200.sharding import pick_best, shard_rows  # noqa: E402
from vinf_3080ti_b200.synth import IQ_SWEEP, LAYER_SET, LM_HEAD, N_LAYERS, synthetic_activations, synthetic_blocks, tensor_bytes  # noqa: E402

METRIC = "quant-matvec weight GB/s, synthetic-27B decode pass"
# DRAM bytes (read + write) of one launch of the dominant kernel (Q3_K 17408 x 5120, M = 4) from an ncu capture
NCU_TRAFFIC_BYTES_PER_LAUNCH = 38447616
SM_COUNT, SM_LANES, SM_MAX_HZ = 148, 128, 1.965e9


# ---- helpers ---------------------------------------------------------------------------------------------

def measured_peaks() -> dict:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)) or None, "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def fma_ceiling_gbs(t: T, m: int) -> float:
    """Weight GB/s at which one fp32 FMA per weight per activation row saturates the fp32 pipe (148 SMs x 128 lanes)."""
    block, size = TRAITS[t]
    return SM_COUNT * SM_LANES * SM_MAX_HZ / m * (size / block) / 1e9


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [v for v in sm if v > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def pass_tensors() -> list[tuple[str, T, int, int]]:
    out = []
    for layer in range(N_LAYERS):
        for name, t, rows, cols in LAYER_SET:
            out.append((f"blk.{layer}.{name}", t, rows, cols))
    out.append((LM_HEAD[0],) + LM_HEAD[1:])
    return out


def codebooks() -> dict[str, bytes]:
    with np.load(REPO / "tests" / "golden" / "iq_codebooks.npz") as z:
        return {k: z[k].tobytes() for k in z.files}


# ---- the CPU arm -----------------------------------------------------------------------------------------

def cpu_weights(distinct: int = 4) -> dict:
    """Host copies of `distinct` layer sets and the LM head (seeded synthetic blocks)."""
    rng = np.random.default_rng(0)
    sets = [[(name, t, rows, cols, synthetic_blocks(t, rows, cols, rng)) for name, t, rows, cols in LAYER_SET] for _ in range(distinct)]
    name, t, rows, cols = LM_HEAD
    return {"sets": sets, "head": (name, t, rows, cols, synthetic_blocks(t, rows, cols, rng))}


class CpuArm:
    """The reference's own CPU matvec (oracle/_ref, compiled from the reference's qwen_cpu.c) on the pass's byte mix: the
    seven tensors of a layer 64 times, then the Q6_K LM head once.  Several distinct layer sets are held in memory and
    taken in turn, so that consecutive layers do not find their weights in the host's caches.  Falls back to the
    plain-C oracle port (OpenMP over rows) only if the reference build is missing."""

    def __init__(self, m: int, threads: int, weights: dict, layers: int = N_LAYERS) -> None:
        from tests import oracle_libs

        self.m, self.layers = m, layers
        mod = oracle_libs.load_reference_cpu_module()
        self.kind = "reference" if mod is not None else "port"
        rng = np.random.default_rng(1)
        sets, head = weights["sets"], weights["head"]
        distinct = len(sets)
        self.nbytes = layers * sum(tensor_bytes(t, r, c) for _, t, r, c in LAYER_SET) + tensor_bytes(*LM_HEAD[1:])
        xs = {name: synthetic_activations(m, cols, rng) for name, _, _, cols in LAYER_SET}
        x_head = synthetic_activations(m, head[3], rng)
        if mod is not None:
            rt = mod.CpuRuntime(codebooks()["iq3s_grid"], threads)
            self.threads_used = threads if threads > 0 else max(1, (os.cpu_count() or 2) // 2)  # its default: half the processors
            self.keep = []
            for name, t, rows, cols in LAYER_SET:
                rt.alloc(f"{name}.x", m * cols)
                rt.alloc(f"{name}.y", m * rows)
                rt.write(f"{name}.x", xs[name].tobytes())
            for k, layer_set in enumerate(sets):
                for name, t, rows, cols, raw in layer_set:
                    data = raw.tobytes()
                    self.keep.append(data)
                    rt.add_tensor(f"{k}.{name}", data, int(t), cols, rows)
            name, t, rows, cols, raw = head
            data = raw.tobytes()
            self.keep.append(data)
            rt.add_tensor(name, data, int(t), cols, rows)
            rt.alloc("lm.x", m * cols)
            rt.alloc("lm.y", m * rows)
            rt.write("lm.x", x_head.tobytes())

            def one_pass() -> None:
                for layer in range(layers):
                    k = layer % distinct
                    for tname, *_ in LAYER_SET:
                        rt.qmv(f"{k}.{tname}", f"{tname}.x", f"{tname}.y", m)
                rt.qmv(LM_HEAD[0], "lm.x", "lm.y", m)
        else:
            clib = oracle_libs.load_c_oracle()
            self.threads_used = os.cpu_count() or 1

            def one_pass() -> None:
                for layer in range(layers):
                    for name, t, rows, cols, raw in sets[layer % distinct]:
                        oracle_libs.c_qmv(clib, raw, int(t), rows, cols, xs[name])
                name, t, rows, cols, raw = head
                oracle_libs.c_qmv(clib, raw, int(t), rows, cols, x_head)

        self._pass = one_pass
        self.sample = (f"the pass's byte mix at M={m}: {layers} x (Q6_K q/k/v/o, Q3_K gate/up, Q4_K down; {distinct} distinct layer sets in turn) "
                       f"+ the Q6_K LM head, {self.nbytes} weight bytes per step")

    def one_pass(self) -> float:
        t0 = time.perf_counter()
        self._pass()
        return time.perf_counter() - t0


def cpu_baseline(m: int, seconds: float) -> dict:
    """The reference CPU path on a bounded number of passes: all host threads, then the reference's own default
    (half the processors, engine/csrc/cpu/qwen_cpu.c:438) for a few passes beside it."""
    nproc = os.cpu_count() or 1
    weights = cpu_weights()
    arm = CpuArm(m, nproc, weights)
    arm.one_pass()
    times = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end or len(times) < 2:
        times.append(arm.one_pass())
    out = {"value": arm.nbytes / min(times) / 1e9, "median": arm.nbytes / statistics.median(times) / 1e9, "unit": "GB/s", "cores": arm.threads_used,
           "kind": arm.kind, "sample": f"{arm.sample}; best (value) and median of {len(times)} passes in ~{seconds:.0f} s"}
    if arm.kind == "reference":
        del arm
        half = CpuArm(m, 0, weights)
        half.one_pass()
        ht = [half.one_pass() for _ in range(3)]
        out["reference_default_threads"] = {"value": half.nbytes / min(ht) / 1e9, "median": half.nbytes / statistics.median(ht) / 1e9,
                                            "cores": half.threads_used, "note": "threads = 0: the reference's default, half the processors"}
    return out


def run_reference(args) -> None:
    """--impl reference: the reference's CPU implementation of the path on this host's cores.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    nproc = os.cpu_count() or 1
    arm = CpuArm(args.m, nproc, cpu_weights())
    warmup = max(1, args.warmup)
    for _ in range(warmup):
        arm.one_pass()
    times = [arm.one_pass() for _ in range(args.steps)]
    ms = 1e3 * sum(times) / len(times)
    value = arm.nbytes / (ms * 1e-3) / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 outputs; the reference CPU kernel rounds activations to int8 per 32 elements", "data": "synthetic",
        "config": {"workload": f"synthetic-27B decode pass at M={args.m}: {arm.sample}", "activation_rows": args.m},
        "tokens_per_s": args.m / (ms * 1e-3),
        "cpu_baseline": {"value": value, "median": arm.nbytes / statistics.median(times) / 1e9, "best": arm.nbytes / min(times) / 1e9, "unit": "GB/s",
                         "cores": arm.threads_used, "kind": arm.kind, "sample": arm.sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---- single kernels, the prompt GEMM and the reference's CUDA kernel (rank 0 of a one-GPU run) ---------------------

KERNEL_CASES = [(T.Q4_K, 17408, 5120, (1, 4, 8)), (T.Q6_K, 6144, 5120, (1, 4, 8)), (T.IQ4_XS, 17408, 5120, (1, 4, 8)), (T.Q3_K, 17408, 5120, (1, 4, 8))] + \
               [(t, r, c, (1, 8)) for t, r, c in IQ_SWEEP if t is not T.IQ4_XS]


def device_blocks(torch, t: T, rows: int, cols: int, gen, dev):
    """Seeded synthetic raw blocks of a rows x cols tensor, generated on the device (+256 bytes of readable padding)."""
    block, size = TRAITS[t]
    nblk = rows * (cols // block)
    raw = torch.randint(0, 256, (nblk * size + 256,), dtype=torch.uint8, device=dev, generator=gen)
    blocks = raw[: nblk * size].view(nblk, size)
    for off in F16_FIELDS[t]:
        scale = torch.empty(nblk, dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=gen).to(torch.float16)
        blocks[:, off : off + 2] = scale.view(torch.uint8).view(nblk, 2)
    return raw, nblk * size


def time_events(torch, stream, fn, reps: int) -> list[float]:
    out = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        stream.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def kernel_table(rt, torch, stream, dev, peaks: dict) -> list[dict]:
    """Every case: a CUDA graph of one launch per distinct copy of the tensor (more than 2 x L2 of weights in all), CUDA
    events around the graph, best and median of 7 after 3 warm-up replays."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    rows_out = []
    for t, rows, cols, ms in KERNEL_CASES:
        nbytes = tensor_bytes(t, rows, cols)
        copies = max(8, -(-300_000_000 // nbytes))
        keep = []
        for i in range(copies):
            raw, _ = device_blocks(torch, t, rows, cols, gen, dev)
            keep.append(raw)
            rt.bind_tensor(f"k{i}", raw.data_ptr(), int(t), cols, rows)
        x = torch.randn(8 * cols, dtype=torch.float32, device=dev, generator=gen)
        y = torch.empty(8 * rows, dtype=torch.float32, device=dev)
        rt.bind("kx", x.data_ptr(), 8 * cols)
        rt.bind("ky", y.data_ptr(), 8 * rows)
        for m in ms:
            rt.qmv("k0", "kx", "ky", m)  # first use outside of capture
            rt.synchronize()
            rt.capture_begin()
            for i in range(copies):
                rt.qmv(f"k{i}", "kx", "ky", m)
            graph = rt.capture_end()
            for _ in range(3):
                rt.graph_launch(graph)
            times = time_events(torch, stream, lambda: rt.graph_launch(graph), 7)
            rt.graph_destroy(graph)
            us = min(times) * 1e3 / copies
            gbs = nbytes / us / 1e3
            ceiling = min(peaks["hbm_gbs"], fma_ceiling_gbs(t, m))
            rows_out.append({"tensor": f"{t.name} {rows}x{cols}", "M": m, "us": round(us, 2), "us_median": round(statistics.median(times) * 1e3 / copies, 2),
                             "weight_GBs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4), "frac_of_8TBs": round(gbs / 8000.0, 4),
                             "frac_of_min_hbm_fma": round(gbs / ceiling, 4), "copies": copies})
        for i in range(copies):
            rt.free(f"k{i}")
        rt.release("kx")
        rt.release("ky")
        del keep, x, y
    return rows_out


def prefill_gemm(rt, torch, stream, dev, peaks: dict) -> dict:
    """The prompt pass: Q4_K 17408 x 5120 with 512 activation rows through the tensor-core GEMM (set_gemm_min_rows)."""
    t, rows, cols, ntok = T.Q4_K, 17408, 5120, 512
    gen = torch.Generator(device=dev)
    gen.manual_seed(512)
    raw, _ = device_blocks(torch, t, rows, cols, gen, dev)
    rt.bind_tensor("pw", raw.data_ptr(), int(t), cols, rows)
    x = torch.randn(ntok * cols, dtype=torch.float32, device=dev, generator=gen)
    y = torch.empty(ntok * rows, dtype=torch.float32, device=dev)
    rt.bind("px", x.data_ptr(), ntok * cols)
    rt.bind("py", y.data_ptr(), ntok * rows)
    rt.set_gemm_min_rows(64)
    try:
        for _ in range(3):
            rt.qmv("pw", "px", "py", ntok)
        rt.synchronize()
        times = time_events(torch, stream, lambda: rt.qmv("pw", "px", "py", ntok), 7)
    finally:
        rt.set_gemm_min_rows(0)
    rt.free("pw")
    rt.release("px")
    rt.release("py")
    ms = min(times)
    flops = 2.0 * ntok * rows * cols
    return {"tensor": f"{t.name} {rows}x{cols}", "activation_rows": ntok, "ms": round(ms, 4), "ms_median": round(statistics.median(times), 4),
            "TFLOPs": round(flops / ms / 1e9, 1), "frac_of_bf16_burst": round(flops / ms / 1e9 / peaks["bf16_tflops"], 4),
            "frac_of_bf16_sustained": round(flops / ms / 1e9 / peaks["bf16_tflops_sustained"], 4) if peaks.get("bf16_tflops_sustained") else None,
            "note": "fp32 activations -> fp16; pairs of blocks on tcgen05.mma.cta_group::2, each 128 weight rows x 512 activation rows with fp32 "
                    "accumulators in tensor memory; weights: raw blocks staged in shared memory by bulk copies, per-block decoders to fp16 "
                    "tiles; activations: TMA tile copies; "
                    "time includes the fp32 -> fp16 conversion of the activations"}


def reference_cuda_kernels(torch, dev, ours: list[dict]) -> dict:
    """The reference's own CUDA matvec kernel (its qwen_runtime.cu compiled unchanged for sm_100a into oracle/_ref), launched by
    its own runtime on its stream, on the four main tensors at M = 1 / 4 / 8 over 4 distinct copies (> L2)."""
    import importlib.util

    path = REPO / "oracle" / "_ref" / "_cuda_qwen_runtime.so"
    if not path.exists():
        return {"unavailable": "oracle/_ref/_cuda_qwen_runtime.so has not been built"}
    spec = importlib.util.spec_from_file_location("_cuda_qwen_runtime", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    ref = mod.Runtime(codebooks()["iq3s_grid"])
    stream = torch.cuda.default_stream()  # the reference launches on the legacy default stream
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    mine = {(r["tensor"], r["M"]): r["us"] for r in ours}
    out = []
    for t, rows, cols, ms in KERNEL_CASES[:4]:
        nbytes = tensor_bytes(t, rows, cols)
        copies = max(4, -(-160_000_000 // nbytes))
        for i in range(copies):
            raw, n = device_blocks(torch, t, rows, cols, gen, dev)
            ref.upload(f"w{i}", raw[:n].cpu().numpy().tobytes(), int(t), cols, rows)
        ref.alloc("x", 8 * cols)
        ref.alloc("y", 8 * rows)
        ref.write("x", synthetic_activations(8, cols, np.random.default_rng(1)).tobytes())
        for m in ms:
            def run() -> None:
                for i in range(copies):
                    ref.qmv(f"w{i}", "x", "y", m)
            run()
            ref.synchronize()
            times = time_events(torch, stream, run, 4)
            us = min(times) * 1e3 / copies
            row = {"tensor": f"{t.name} {rows}x{cols}", "M": m, "us": round(us, 2), "weight_GBs": round(nbytes / us / 1e3, 1)}
            if (row["tensor"], m) in mine:
                row["this_library_us"] = mine[(row["tensor"], m)]
                row["this_library_speedup"] = round(us / mine[(row["tensor"], m)], 2)
            out.append(row)
        for i in range(copies):
            ref.free(f"w{i}")
    return {"kernel": "vinf_qmatvec_kernel (engine/csrc/megakernel/qwen_runtime.cu:579-628), unchanged source, -arch=sm_100a", "rows": out}


# ---- the GPU arm -----------------------------------------------------------------------------------------

def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from vinf_3080ti_b200.runtime import Runtime

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    m = args.m
    books = codebooks()
    rt = Runtime(books["iq3s_grid"], books)
    # the runtime launches on a stream torch owns, so that torch events, copies and NCCL order against it
    stream = torch.cuda.Stream(device=dev)
    rt.set_stream(stream.cuda_stream)
    peaks = measured_peaks()

    # -- weights: seeded synthetic blocks generated on the device, this rank's row slice of every tensor
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    keep = []
    weight_bytes_total = 0
    tensors = pass_tensors()
    local_rows: dict[str, tuple[int, int]] = {}
    for name, t, rows, cols in tensors:
        begin, end = shard_rows(rows, rank, world)
        raw, _ = device_blocks(torch, t, end - begin, cols, gen, dev)
        keep.append(raw)
        rt.bind_tensor(name, raw.data_ptr(), int(t), cols, end - begin)
        local_rows[name] = (begin, end)
        weight_bytes_total += tensor_bytes(t, rows, cols)
    rt.set_argmax_row_base(LM_HEAD[0], local_rows[LM_HEAD[0]][0])

    # -- activations and outputs.  The synthetic pass has no ops between the matvecs, so every matvec of a given
    #    input width reads the same activation buffer (the check pass of a multi-GPU run chains them instead).
    widths = sorted({cols for _, _, _, cols in tensors})
    host_x = {w: torch.from_numpy(synthetic_activations(m, w, np.random.default_rng(w))).pin_memory() for w in widths}
    dev_x = {w: torch.empty(m * w, dtype=torch.float32, device=dev) for w in widths}
    for w in widths:
        rt.bind(f"x{w}", dev_x[w].data_ptr(), m * w)
        dev_x[w].copy_(host_x[w].view(-1))

    def kind_of(name: str) -> str:
        return name.split(".")[-1]

    def slice_rows(r: int, k: int) -> int:
        b, e = shard_rows(r, k, world)
        return e - b

    # per kind of tensor: this rank's [M][rows of the slice] block, padded to the widest slice so that one
    # all_gather_into_tensor of equal-sized chunks combines the ranks (NCCL arm and the check)
    kind_rows = {kind_of(name): rows for name, _, rows, _ in tensors}
    widest = {k: max(slice_rows(r, i) for i in range(world)) for k, r in kind_rows.items()}
    y_local = {k: torch.zeros(m * widest[k], dtype=torch.float32, device=dev) for k in kind_rows}
    for k, r in kind_rows.items():
        rt.bind(f"y.{k}", y_local[k].data_ptr(), m * slice_rows(r, rank))
    gathered = {k: torch.empty(world * m * widest[k], dtype=torch.float32, device=dev) for k in kind_rows} if world > 1 else {}
    ids_addr, vals_addr = rt.argmax_result()
    torch.cuda.synchronize()

    # The launches of a pass.  Tensors that read the same activations and share type and columns go out as ONE launch
    # (q/k/v, gate/up) unless --launches per-tensor asks for the reference's one kernel per tensor.
    GROUPS = {"attn_q": 0, "attn_k": 0, "attn_v": 0, "attn_o": 1, "ffn_gate": 2, "ffn_up": 2, "ffn_down": 3, "output": 4}
    launches_of_pass: list[list[tuple[str, T, int, int]]] = []
    for entry in tensors:
        layer, g = entry[0].rsplit(".", 1)[0], GROUPS[kind_of(entry[0])]
        if args.launches == "grouped" and launches_of_pass and launches_of_pass[-1][0][0].rsplit(".", 1)[0] == layer and \
                GROUPS[kind_of(launches_of_pass[-1][0][0])] == g:
            launches_of_pass[-1].append(entry)
        else:
            launches_of_pass.append([entry])

    def enqueue_launch(group, fused_argmax: bool = False) -> None:
        cols = group[0][3]
        if fused_argmax:
            rt.qmv_argmax(group[0][0], f"x{cols}", f"y.{kind_of(group[0][0])}", m, blocking=False)
        elif len(group) == 1:
            rt.qmv(group[0][0], f"x{cols}", f"y.{kind_of(group[0][0])}", m)
        else:
            rt.qmv_group([e[0] for e in group], f"x{cols}", [f"y.{kind_of(e[0])}" for e in group], m)

    def enqueue_pass() -> None:  # this rank's kernels alone: the whole pass on one GPU, the "exchange off" figure on several
        for group in launches_of_pass[:-1]:
            enqueue_launch(group)
        enqueue_launch(launches_of_pass[-1], fused_argmax=True)

    enqueue_pass()  # sets the kernels' attributes outside of capture
    rt.synchronize()
    rt.capture_begin()
    enqueue_pass()
    local_graph = rt.capture_end()

    def nccl_pass() -> None:  # NCCL arm: kernel, all-gather(s), kernel, ... launched eagerly
        for group in launches_of_pass[:-1]:
            enqueue_launch(group)
            for e in group:
                dist.all_gather_into_tensor(gathered[kind_of(e[0])], y_local[kind_of(e[0])])
        enqueue_launch(launches_of_pass[-1], fused_argmax=True)
        dist.all_gather_into_tensor(gathered["output"], y_local["output"])

    # Fused arm (default): every matvec pushes its slice into the gathered vector of every rank from its own epilogue and
    # the next matvec waits for all ranks' flags - the dependency chain of a tensor-parallel decoder.  One gathered
    # vector per kind of tensor (q, k, v, o, gate, up, down, logits); one flag slot per launch of the pass; the whole
    # pass is one CUDA graph per rank and contains no collective.
    use_push = world > 1 and args.gather == "push"
    push_graph = None
    if use_push:
        from vinf_3080ti_b200.sharding import ExchangeLayout, connect_exchange

        kinds = {}
        off = 0
        for name, t, rows, cols in tensors:
            if kind_of(name) not in kinds:
                kinds[kind_of(name)] = off
                off += (4 * m * rows + 255) // 256 * 256
        layout = ExchangeLayout(off, n_slots=len(launches_of_pass))
        region_addrs = connect_exchange(rt, layout)
        for k, at in kinds.items():  # the gathered vectors inside this rank's own region, as buffers
            rt.bind(f"g.{k}", region_addrs[rank] + at, m * kind_rows[k])

        # the launch whose flags a launch waits for: the last one that produced (part of) its input
        producer_kind = {"attn_q": "ffn_down", "attn_o": "attn_v", "ffn_gate": "attn_o", "ffn_up": "attn_o", "ffn_down": "ffn_up",
                         "output": "ffn_down"}
        last_of_kind: dict[str, int] = {}
        wait_for = []
        for i, group in enumerate(launches_of_pass):
            lead = kind_of(group[0][0])
            wait_for.append(last_of_kind.get(producer_kind.get(lead, "ffn_down"), len(launches_of_pass) - 1))  # first layer: previous pass's last launch
            for e in group:
                last_of_kind[kind_of(e[0])] = i

        def push_launch(i: int, x_of: dict | None = None) -> None:
            """Launch i of the pass with its push; x_of maps an input width to the buffer to read instead of the local one."""
            group = launches_of_pass[i]
            cols = group[0][3]
            x_name = (x_of or {}).get(kind_of(group[0][0]), f"x{cols}")  # keyed by the kind of the launch's first tensor
            if len(group) == 1:
                name, t, rows, _ = group[0]
                rt.qmv_push(name, x_name, f"y.{kind_of(name)}", m, slot=i, dst_off=kinds[kind_of(name)], rows_total=rows,
                            row_begin=local_rows[name][0], wait_slot=wait_for[i], with_argmax=(i == len(launches_of_pass) - 1))
            else:
                rt.qmv_push_group([e[0] for e in group], x_name, [f"y.{kind_of(e[0])}" for e in group], m, slot=i,
                                  dst_offs=[kinds[kind_of(e[0])] for e in group], rows_totals=[e[2] for e in group],
                                  row_begins=[local_rows[e[0]][0] for e in group], wait_slot=wait_for[i])

        def push_pass() -> None:
            for i in range(len(launches_of_pass)):
                push_launch(i)

        push_pass()
        rt.synchronize()
        dist.barrier()
        rt.capture_begin()
        push_pass()
        push_graph = rt.capture_end()

    def device_pass() -> None:
        if world == 1:
            rt.graph_launch(local_graph)
        elif use_push:
            rt.graph_launch(push_graph)
        else:
            with torch.cuda.stream(stream):
                nccl_pass()

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int) -> float:
        """ms per step: CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            tmax = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            ms = float(tmax.item())
        return ms

    # global argmax of a sharded LM head: every rank's (value, index) pairs are all-gathered on the device, one small
    # device -> host copy, then highest value wins, lowest index on ties
    if world > 1:
        pair = torch.zeros((2, 8), dtype=torch.float32, device=dev)   # row 0: values, row 1: the int32 ids' bits
        pairs = torch.zeros((world, 2, 8), dtype=torch.float32, device=dev)
        pairs_host = torch.zeros((world, 2, 8), dtype=torch.float32).pin_memory()
        rt.bind("argmax.pair", pair.data_ptr(), 16)
        rt.bind("argmax.vals", vals_addr, 8)
        rt.bind("argmax.ids", ids_addr, 8)

    def combined_ids() -> list[int]:
        rt.copy("argmax.pair", 0, "argmax.vals", 0, m)
        rt.copy("argmax.pair", 8, "argmax.ids", 0, m)
        with torch.cuda.stream(stream):
            dist.all_gather_into_tensor(pairs, pair)
            pairs_host.copy_(pairs, non_blocking=True)
        stream.synchronize()
        return pick_best(pairs_host[:, 0, :m].to(torch.float64), pairs_host[:, 1, :m].contiguous().view(torch.int32).to(torch.int64)).tolist()

    def e2e_step() -> None:
        with torch.cuda.stream(stream):
            for w in widths:
                dev_x[w].copy_(host_x[w].view(-1), non_blocking=True)
        device_pass()
        if world == 1:
            rt.argmax_fetch(m, with_values=True)
        else:
            combined_ids()

    # The same step through the calls the reference's executor makes on its runtime: write the activations from host
    # memory, one qmv / qmv_group call per launch (no graph), argmax_rows over the stored logits (blocking, ids to the host).
    host_np = {w: host_x[w].numpy() for w in widths}

    def plugin_step() -> None:
        for w in widths:
            rt.write(f"x{w}", host_np[w])
        for group in launches_of_pass:
            enqueue_launch(group)
        rt.argmax_rows("y.output", kind_rows["output"], m)

    # -- warm-up, then the timed regions
    for _ in range(max(3, args.warmup)):
        device_pass()
    launches_before = rt.launch_count()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(device_pass, args.steps)
    launches = rt.launch_count() - launches_before
    e2e_ms = timed(e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    plugin_ms = None
    if world == 1:
        plugin_step()
        plugin_ms = timed(plugin_step, max(2, args.steps // 4))

    # -- multi-GPU: what the exchange costs, and whether what it delivers is right
    scaling_detail = None
    check = None
    if world > 1:
        scaling_detail = {"exchange_off_ms": timed(lambda: rt.graph_launch(local_graph), max(2, args.steps // 2)),
                          "note": "exchange_off: this rank's sharded kernels alone (no push, no waits, one graph)"}
        if use_push:
            def nccl_step() -> None:
                with torch.cuda.stream(stream):
                    nccl_pass()

            nccl_step()
            scaling_detail["nccl_allgather_ms"] = timed(nccl_step, max(2, args.steps // 4))
            check = multi_gpu_check(torch, dist, rt, stream, dev, m, rank, world, launches_of_pass, kind_of, kind_rows, widest, slice_rows,
                                    y_local, gathered, push_launch, combined_ids)

    # -- roofline of the dominant kernel: the Q3_K gate/up matvec alone over the model's distinct tensors
    dom = [(n, t, r, c) for n, t, r, c in tensors if t is T.Q3_K]
    d_rows = local_rows[dom[0][0]][1] - local_rows[dom[0][0]][0]

    def dominant() -> None:
        for name, t, rows, cols in dom:
            rt.qmv(name, f"x{cols}", f"y.{kind_of(name)}", m)

    dominant()
    dom_ms = timed(dominant, max(2, args.steps // 2)) / len(dom)
    alg_bytes = d_rows * (dom[0][3] // 256) * 110 + 4 * m * dom[0][3] + 4 * m * d_rows
    achieved = alg_bytes / (dom_ms * 1e-3) / 1e9
    fma_ceiling = fma_ceiling_gbs(T.Q3_K, m)

    if rank == 0:
        value = weight_bytes_total / (ms * 1e-3) / 1e9
        e2e_value = weight_bytes_total / (e2e_ms * 1e-3) / 1e9
        h2d = sum(4 * m * w for w in widths)
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"synthetic-27B decode pass, M={m}: 64 x (Q6_K q/k/v/o, Q3_K gate/up, Q4_K down) + Q6_K LM head 151936x5120 "
                                   f"with fused argmax; {weight_bytes_total} weight bytes resident in HBM", "activation_rows": m,
                       "launches_per_pass": len(launches_of_pass), "launches": args.launches, "l2": "pass is ~100x larger than L2 (no flush needed)",
                       "parallelism": "single GPU, one CUDA graph per pass" if world == 1 else (f"output rows sharded over {world} GPUs; every matvec pushes its slice into all ranks' gathered vector over NVLink from its epilogue "
                                        "and waits for the flags of the launch that produced its input (decoder dependency chain); one CUDA graph per rank, no collective" if use_push else
                                        f"output rows sharded over {world} GPUs, NCCL all-gather after every matvec, eager launches")},
            "tokens_per_s": m / (ms * 1e-3), "pct_of_8TBs": 100.0 * value / 8000.0 / world,
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 * m if world == 1 else 64 * world,
                    "tokens_per_s": m / (e2e_ms * 1e-3)},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if (m == 4 and world == 1) else None, "kernel": f"qmv_kernel<Q3_K, M={m}> {d_rows}x{dom[0][3]}",
                         "algorithmic_bytes_per_launch": alg_bytes, "us_per_launch": dom_ms * 1e3, "peak_source": f"of {peaks['source']}",
                         "fp32_fma_ceiling": {"weight_GBs": fma_ceiling, "frac": achieved / min(peaks["hbm_gbs"], fma_ceiling),
                                              "note": "achieved / min(HBM peak, rate at which one FMA per weight per activation row saturates the fp32 pipe)"}},
            "clocks": clocks,
        }
        if plugin_ms is not None:
            line["e2e"]["plugin_calls"] = {"value": weight_bytes_total / (plugin_ms * 1e-3) / 1e9, "ms_per_step": plugin_ms,
                                           "calls": "write x3, qmv / qmv_group x257, argmax_rows (blocking): one call per launch, no graph, "
                                                    "activations from host memory, ids to the host",
                                           "d2h_bytes_per_step": 4 * m}
        if scaling_detail is not None:
            line["scaling_detail"] = scaling_detail
        if check is not None:
            line["multi_gpu_check"] = check
        if world == 1 and not args.no_extras:
            for key, fn in (("kernels", lambda: kernel_table(rt, torch, stream, dev, peaks)), ("prefill", lambda: prefill_gemm(rt, torch, stream, dev, peaks))):
                try:  # the extra legs never take the measurement down with them
                    line[key] = fn()
                except Exception as exc:
                    line[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            try:
                line["reference_cuda_kernel"] = reference_cuda_kernels(torch, dev, line["kernels"] if isinstance(line.get("kernels"), list) else [])
            except Exception as exc:
                line["reference_cuda_kernel"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        if world == 1 and args.cpu_seconds > 0:
            line["cpu_baseline"] = cpu_baseline(m, args.cpu_seconds)
        print(json.dumps(line))
    torch.cuda.synchronize()
    ok = check is None or bool(check.get("ok"))
    rt.set_stream(None)
    rt.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        sys.exit(3)


def multi_gpu_check(torch, dist, rt, stream, dev, m, rank, world, launches_of_pass, kind_of, kind_rows, widest, slice_rows, y_local, gathered,
                    push_launch, combined_ids) -> dict:
    """One CHAINED layer after the timed regions: every consumer reads the gathered vector that the pushes of its
    producer left in this rank's exchange region (down from the local activations, then q/k/v <- down, o <- q,
    gate/up <- o, down <- up, LM head <- down; the widths match), so the peer stores, the flags and the bounded waits
    are what the data goes through.  Run twice: launch by launch with a barrier in between, then back to back with no
    host synchronisation at all (the ranks' kernels really wait for one another).  On every rank, after each: (a) each
    gathered vector equals an NCCL all-gather of the ranks' local slices bit for bit, (b) the combined argmax ids equal
    the argmax (lowest index on ties) of the all-gathered logits."""
    chain_input = {"attn_q": "g.ffn_down", "attn_k": "g.ffn_down", "attn_v": "g.ffn_down", "attn_o": "g.attn_q", "ffn_gate": "g.attn_o",
                   "ffn_up": "g.attn_o", "ffn_down": "g.ffn_up", "output": "g.ffn_down"}
    n = len(launches_of_pass)
    layer0 = [i for i in range(n) if launches_of_pass[i][0][0].startswith("blk.0.")]
    down = next(i for i in layer0 if kind_of(launches_of_pass[i][0][0]) == "ffn_down")
    order = [(down, False)] + [(i, True) for i in layer0] + [(n - 1, True)]  # (launch, input from the exchange region)

    def gathered_reference(kind: str):
        """[M][rows] assembled from an NCCL all-gather of the ranks' local [M][slice] blocks."""
        with torch.cuda.stream(stream):
            dist.all_gather_into_tensor(gathered[kind], y_local[kind])
        stream.synchronize()
        parts = gathered[kind].view(world, -1)
        return torch.cat([parts[k][: m * slice_rows(kind_rows[kind], k)].view(m, -1) for k in range(world)], dim=1).contiguous()

    def region_vector(kind: str):
        addr, count = rt.buffer_ptr(f"g.{kind}")
        got = torch.empty(count, dtype=torch.float32, device=dev)
        rt.bind("check.tmp", got.data_ptr(), count)
        rt.copy("check.tmp", 0, f"g.{kind}", 0, count)
        rt.synchronize()
        rt.release("check.tmp")
        return got.view(m, -1)

    def verify(label: str, mismatches: list) -> None:
        for kind in kind_rows:
            ref = gathered_reference(kind)
            if not torch.equal(region_vector(kind).view(torch.int32), ref.view(torch.int32)):
                mismatches.append(f"{label}: the pushed {kind} vector differs from the all-gather of the slices")
            if not torch.isfinite(ref).all():
                mismatches.append(f"{label}: non-finite {kind} outputs")
        ids = [int(v) for v in combined_ids()]
        want = [int(v) for v in torch.argmax(gathered_reference("output"), dim=1).tolist()]
        if ids != want:
            mismatches.append(f"{label}: combined argmax {ids} != argmax of the gathered logits {want}")

    mismatches: list[str] = []
    for label, stepwise in (("launch by launch", True), ("back to back", False)):
        for i, chained in order:
            push_launch(i, chain_input if chained else None)
            if stepwise:
                rt.synchronize()
                dist.barrier()
        rt.synchronize()
        dist.barrier()
        verify(label, mismatches)
        dist.barrier()
    flag = torch.tensor([len(mismatches)], dtype=torch.int64, device=dev)
    dist.all_reduce(flag)
    return {"ok": int(flag.item()) == 0, "n_ranks": world, "launches_chained": len(order), "this_rank_mismatches": mismatches[:4],
            "what": "a chained layer + LM head through the exchange regions, launch by launch and then back to back without host synchronisation: "
                    "pushed vectors == NCCL all-gather of the slices (bitwise) on every rank; combined argmax ids == argmax of the all-gathered logits"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--m", type=int, default=4, help="activation rows per pass (1..8)")
    ap.add_argument("--launches", default="grouped", choices=["grouped", "per-tensor"],
                    help="grouped: q/k/v and gate/up of a layer go out as one launch each; per-tensor: one kernel per tensor, as the reference launches")
    ap.add_argument("--gather", default="push", choices=["push", "nccl"],
                    help="multi-GPU: how output slices are combined - fused peer-memory push from the kernel (default) or NCCL all-gather")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="seconds of CPU work for the cpu_baseline leg (0 = skip)")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-kernel table, the prompt GEMM and the reference's CUDA kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
