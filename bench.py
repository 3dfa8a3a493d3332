"""Benchmark of the realizer-bridge forward hot path on B200.

Workload (``config.workload``): configuration 2 of the baseline, the fused elementwise/reduce
chains over fp32 [16384, 4096] tensors -- one step = three realizations through the bridge,
``y = relu(a*b+c)*exp(-d)``, ``y.sum(-1)`` and ``softmax(y, -1)`` -- on seeded N(0,1) inputs.
``value`` is algorithmic HBM GB/s with the inputs already resident in HBM; ``e2e`` is the same
metric through ``realize_cuda`` with pinned host buffers (host<->device copies inside the timed
region).  Algorithmic bytes per step: (4 reads + 1 write) * 4 B * R*C for y and for the softmax,
4 reads * 4 B * R*C + 4 B * R for the row sum.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Under torchrun every rank runs its own shard of the same size (weak scaling, no data-path
collective); the timed region is bracketed by a barrier + synchronize and the slowest rank's
device time is used.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 16384, 4096
METRIC = "fused-eltwise HBM GB/s, GEMM TFLOP/s, attention tok/s at 1/2/4/8 B200 vs roofline"
# the same string in both arms; how many of the rows one step covers is a key of its own (rows_per_step)
WORKLOAD = f"config 2: fused elementwise/reduce chains y, row-sum, row-softmax over fp32 [{ROWS},{COLS}]"


def algorithmic_bytes(rows: int, cols: int) -> dict:
    rc = rows * cols
    return {"y": 20 * rc, "rowsum": 16 * rc + 4 * rows, "rowsoftmax": 20 * rc}


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.source = "nvidia-smi"
        self._stop_evt = threading.Event()

    def _sample_nvml(self, nv, handle) -> None:
        self.samples.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
        self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
        bits = nv.nvmlDeviceGetCurrentClocksEventReasons(handle) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
            else nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
        for name, mask in (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40),
                           ("sw_power_cap", 0x4)):
            if bits & mask:
                self.reasons.add(name)

    def _sample_smi(self) -> None:
        out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                              "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
        parts = [p.strip() for p in out.split(",")]
        if len(parts) >= 6:
            self.samples.append(float(parts[0]))
            self.max_mhz = float(parts[1])
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    self.reasons.add(name)

    def run(self) -> None:
        # read-only queries: NVML in-process (about a millisecond each) when the module is there,
        # else one nvidia-smi process per sample
        nv = handle = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.source = "nvml"
        except Exception:
            nv = None
            self.source = "nvidia-smi"
        while not self._stop_evt.is_set():
            try:
                if nv is not None:
                    self._sample_nvml(nv, handle)
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop_evt.wait(0.01 if nv is not None else 0.1)

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=6)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
                "source": self.source}


def build_graphs(graph, configs, arrays):
    store = graph.BufferStore()
    t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
    return store, t, {"y": configs.chain_y(graph, t), "rowsum": configs.chain_rowsum(graph, t),
                      "rowsoftmax": configs.chain_rowsoftmax(graph, t)}


def cpu_reference_realize():
    """Returns (kind, realize(build, arrays) -> seconds).  Uses the unmodified reference realizer
    when ``oracle/_ref`` travelled with the tree, else the NumPy restatement in ``oracle/port.py``."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if os.path.isdir(os.path.join(ref_dir, "browsergrad_jit")):
        sys.path.insert(0, ref_dir)
        try:
            import browsergrad_jit as bg
            from oracle.ref_api import RefApi
            api = RefApi(bg)

            def run(arrays):
                from browsergrad_b200 import configs
                t = {k: bg.from_numpy(v) for k, v in arrays.items()}
                t0 = time.perf_counter()
                configs.chain_y(api, t).numpy()
                configs.chain_rowsum(api, t).numpy()
                configs.chain_rowsoftmax(api, t).numpy()
                return time.perf_counter() - t0
            return "reference", run
        except Exception:
            pass
    from browsergrad_b200 import configs, graph, passes
    from oracle import port

    def run(arrays):
        store, t, roots = build_graphs(graph, configs, arrays)
        prepared = {k: passes.prepare(v._uop) for k, v in roots.items()}
        t0 = time.perf_counter()
        for k in ("y", "rowsum", "rowsoftmax"):
            port.realize(prepared[k], store)
        return time.perf_counter() - t0
    return "port", run


def _cpu_worker(index: int, sample_rows: int, warmup: int, steps: int, gate) -> None:
    """One host process of the CPU arm: realizes its own row block of the workload once per step.
    NumPy's ufuncs and reductions run on one thread, so the reference's path uses all host cores
    only when its rows are split over processes -- the same split the GPUs get."""
    from browsergrad_b200 import configs
    _, run = cpu_reference_realize()
    arrays = configs.chain_inputs(sample_rows, COLS)
    if index:
        arrays = {k: np.roll(v, index, axis=0) for k, v in arrays.items()}
    for _ in range(warmup):
        run(arrays)
    for _ in range(steps):
        gate.wait()
        run(arrays)
        gate.wait()


def cpu_reference_steps(sample_rows: int, workers: int, warmup: int, steps: int) -> list:
    """Wall-clock seconds of each of ``steps`` concurrent passes of ``workers`` processes."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")      # never fork a process that may hold a CUDA context
    gate = ctx.Barrier(workers + 1)
    procs = [ctx.Process(target=_cpu_worker, args=(i, sample_rows, warmup, steps, gate), daemon=True) for i in range(workers)]
    for pr in procs:
        pr.start()
    times = []
    try:
        for _ in range(steps):
            gate.wait(timeout=600)
            t0 = time.perf_counter()
            gate.wait(timeout=600)
            times.append(time.perf_counter() - t0)
    finally:
        for pr in procs:
            pr.join(timeout=30)
            if pr.is_alive():
                pr.terminate()
    return times


def cpu_baseline(sample_rows: int, repeats: int = 1) -> dict:
    from browsergrad_b200 import configs
    kind, run = cpu_reference_realize()
    arrays = configs.chain_inputs(sample_rows, COLS)
    run(arrays)  # warm-up
    single = min(run(arrays) for _ in range(max(1, repeats)))
    nbytes = sum(algorithmic_bytes(sample_rows, COLS).values())
    workers = os.cpu_count() or 1
    times = cpu_reference_steps(sample_rows, workers, 1, max(2, repeats))
    best = min(times)
    return {"value": workers * nbytes / best / 1e9, "unit": "GB/s", "cores": workers, "kind": kind,
            "sample": f"{workers} processes x {sample_rows} of {ROWS} rows x {COLS} cols each, all three realizations, "
                      f"NumPy {np.__version__}, best of {max(2, repeats)} after 1 warm-up",
            "seconds": best, "single_process_value": nbytes / single / 1e9}


EXTRA_WARMUP = 3   # untimed realizations before each extra workload; a profiler capture lowers it (--extra-warmup)


def time_plan(bridge, torch, stream, graph_root, store, front, steps: int, warmup: int = -1):
    """Average device time (ms) of one realization with resident leaves, plus the per-kernel profile.
    The plan is timed without per-unit events; the profile comes from runs with them.  Blocks of timed runs
    alternate with single profiled runs, so that both see the same clocks (a long run of GEMMs settles from its burst clock
    to the sustained one: a profile taken only after the timed steps reported units slower than their whole plan)."""
    prepared, plan = front.plan_for(graph_root._uop)
    table = front.DeviceBufferTable(bridge)
    inputs = front._bind_inputs(plan, store, table, True)
    for _ in range(EXTRA_WARMUP if warmup < 0 else warmup):
        bridge.release(bridge.run_tensor_plan_resident(plan, inputs, prepared.dtype))
    bridge.synchronize()
    bridge.flushProfiles()
    n_blocks = max(1, min(steps, 5))
    per = (steps + n_blocks - 1) // n_blocks
    pairs = []
    for _ in range(n_blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(per):
            bridge.release(bridge.run_tensor_plan_resident(plan, inputs, prepared.dtype))
        e1.record(stream)
        pairs.append((e0, e1))
        bridge.set_option("profiling", 1)      # one profiled run per block
        bridge.release(bridge.run_tensor_plan_resident(plan, inputs, prepared.dtype))
        bridge.set_option("profiling", 0)
    bridge.synchronize()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in pairs) / (n_blocks * per)
    prof = bridge.flushProfiles()
    for p in prof:
        p["runs"] = n_blocks                # forwards the profile covers
    trace = bridge.last_plan_trace()
    table.release_all()
    return ms, prof, trace


EXTRA_NAMES = ("mlp", "interp", "ce", "gemm_bf16_1024", "gemm_fp32_1024", "gemm_bf16_4096", "gemm_fp32_4096", "gemm_bf16_8192",
               "gemm_fp32_8192", "attn_fp32", "attn_bf16", "gpt")
NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0}   # B200 data-sheet figures, printed beside the measured peaks


def rows_for_interp(attn_batch: int) -> int:
    """Rows of the interpreter extras: the full 16384 of config 2, scaled down with --attn-batch for profiler captures."""
    return ROWS if attn_batch >= 16 else max(1024, ROWS * attn_batch // 16)


def extra_measurements(bridge, torch, stream, peaks, steps: int, only=None, attn_batch: int = 16) -> dict:
    """Configs 3, 4 and 5 of the baseline: Linear+bias+GELU GEMM TFLOP/s, causal attention tokens/s and
    the GPT decoder forward (one GPU's shard: batch 8) tokens/s.  ``only`` restricts the set (used
    when a single kernel is captured under a profiler)."""
    from browsergrad_b200 import configs, front, graph
    want = set(only) if only else set(EXTRA_NAMES)
    out = {"mlp": [], "interpreter": [], "cross_entropy": [], "gemm": [], "attention": [], "gpt": []}
    if "interp" in want:
        # The generic interpreter, which every fusion group without a specialised kernel gets: the three config-2
        # plans with the pattern kernels switched off, and two chains no pattern matches (an fp32 select chain and the
        # float64 GELU tail the reference's F.gelu produces under NumPy 2).  Algorithmic bytes = operands read once,
        # result written once.
        rows_i = rows_for_interp(attn_batch)
        arrays = configs.chain_inputs(rows_i, COLS)
        store = graph.BufferStore()
        t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
        rc = rows_i * COLS
        plans = [("y = relu(a*b+c)*exp(-d), pattern kernels off", configs.chain_y(graph, t), 20 * rc, 0),
                 ("row-sum of y, pattern kernels off", configs.chain_rowsum(graph, t), 16 * rc + 4 * rows_i, 0),
                 ("row-softmax of y, pattern kernels off", configs.chain_rowsoftmax(graph, t), 20 * rc, 0),
                 ("where(a > b, a*c, d) * exp(-b) + c (fp32, no pattern)",
                  graph.where(t["a"] > t["b"], t["a"] * t["c"], t["d"]) * graph.exp(-t["b"]) + t["c"], 20 * rc, 1),
                 ("gelu(a*b+c) (float64 tail, no pattern)", graph.gelu(t["a"] * t["b"] + t["c"]), (12 + 8) * rc, 1)]
        for name, root, nbytes, keep_patterns in plans:
            bridge.set_option("static_patterns", keep_patterns)
            try:
                ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, steps)
            finally:
                bridge.set_option("static_patterns", 1)
            gbs = nbytes / (ms * 1e-3) / 1e9
            out["interpreter"].append({"workload": f"{name}, fp32 [{rows_i},{COLS}]", "plan_ms": ms, "kernels": trace,
                                       "algorithmic_bytes": nbytes,
                                       "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                                    "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal": gbs / NOMINAL["hbm_gbs"],
                                                    "nominal_peak": NOMINAL["hbm_gbs"], "basis": "plan time"}})
        del arrays, store, t
    if "mlp" in want:
        # configuration 1 is latency-bound (13 MFLOP): report microseconds per forward, no roofline fraction
        arrays = configs.mlp_inputs()
        store = graph.BufferStore()
        t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
        root = configs.mlp_loss(graph, t)
        ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, max(steps, 20))
        out["mlp"].append({"workload": "MLP 784-128(ReLU)-10 + cross entropy, batch 64, fp32", "us_per_forward": ms * 1e3,
                           "kernels": trace,
                           "kernel_us": {p["name"]: 1e3 * p["ms"] / p["runs"] for p in prof},
                           "note": "us_per_forward is the time between back-to-back forwards on the stream (host submission "
                                   "included when it is the slower side); kernel_us are the units' own device times"})
        del arrays, store, t
    if "ce" in want:
        # cross entropy over the vocabulary of configuration 5: [8192, 32000] fp32 logits, int64 targets, mean
        # reduction.  Algorithmic bytes = the logits read once plus the targets.
        import numpy as np
        ce_rows, ce_classes = 8192 * attn_batch // 16 if attn_batch < 16 else 8192, 32000
        rng = np.random.default_rng(5)
        store = graph.BufferStore()
        logits = graph.from_numpy(rng.standard_normal((ce_rows, ce_classes), dtype=np.float32), store)
        target = graph.from_numpy(rng.integers(0, ce_classes, (ce_rows,), dtype=np.int64), store)
        for name, root in (("mean", graph.cross_entropy(logits, target)),
                           ("mean, label smoothing 0.1", graph.cross_entropy(logits, target, label_smoothing=0.1))):
            ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, steps)
            nbytes = ce_rows * ce_classes * 4 + ce_rows * 8
            gbs = nbytes / (ms * 1e-3) / 1e9
            out["cross_entropy"].append({"workload": f"cross entropy ({name}), fp32 logits [{ce_rows},{ce_classes}], int64 targets",
                                         "plan_ms": ms, "kernels": trace, "algorithmic_bytes": nbytes,
                                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                                      "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal": gbs / NOMINAL["hbm_gbs"],
                                                      "nominal_peak": NOMINAL["hbm_gbs"], "basis": "plan time"}})
        del store, logits, target
    for n in (1024, 4096, 8192):
        for amp in ("bfloat16", ""):
            if f"gemm_{'bf16' if amp else 'fp32'}_{n}" not in want:
                continue
            arrays = configs.linear_inputs(n, n, n)
            store = graph.BufferStore()
            t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
            root = configs.linear_gelu(graph, t, amp)
            ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, steps)
            gemm = [p for p in prof if p["name"].startswith("gemm")]
            k_ms = gemm[0]["ms"] / max(gemm[0]["launches"], 1) if gemm else ms
            # the headline rate divides by the whole plan (activation conversion or hi/lo split included: work the
            # graph asks for); the GEMM unit alone, from the profiled pass, is kept beside it
            tf = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
            tf_kernel = 2.0 * n ** 3 / (k_ms * 1e-3) / 1e12
            # fp32 operands: one product on the tf32 path (half the bf16 rate) plus two correction products on the
            # bf16 path = four bf16-product times per result
            peak = peaks["bf16_tflops"] if amp else peaks["bf16_tflops"] / 4.0
            nominal = NOMINAL["bf16_tflops"] if amp else NOMINAL["bf16_tflops"] / 4.0
            out["gemm"].append({"workload": f"Linear+bias+GELU M=N=K={n} {'bf16 autocast' if amp else 'fp32 (3xTF32)'}",
                                "tflops": tf, "plan_ms": ms, "kernel_ms": k_ms, "kernel_tflops": tf_kernel, "kernels": trace,
                                "timing": "plan_ms: CUDA events around back-to-back plans; kernel_ms: events around the GEMM "
                                          "unit in a second, profiled pass (each unit bracketed by events, so units do not overlap)",
                                "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                                             "frac_of_nominal": tf / nominal, "nominal_peak": nominal, "basis": "plan time",
                                             "kernel_only_frac": tf_kernel / peak, "kernel_only_frac_of_nominal": tf_kernel / nominal,
                                             "peak_note": "measured cuBLAS bf16 burst" if amp else
                                             "measured bf16 burst / 4 (split product: tf32(x).tf32(y) at half the bf16 rate "
                                             "plus two bf16 correction products); the three-tf32-pass scheme it replaces had burst / 6"}})
            del arrays, store, t
    b, h, s, d = attn_batch, 12, 2048, 64
    for amp in ("", "bfloat16"):
        if f"attn_{'bf16' if amp else 'fp32'}" not in want:
            continue
        arrays = configs.attention_inputs(b, h, s, d)
        arrays["mask"] = configs.causal_mask(s)
        store = graph.BufferStore()
        t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
        root = configs.attention(graph, t, "mask", amp)
        ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, steps)
        att = [p for p in prof if p["name"].startswith("attention")]
        k_ms = att[0]["ms"] / max(att[0]["launches"], 1) if att else ms
        flops = 4.0 * b * h * s * s * d                     # both products over the full S x S score matrix
        useful = 4.0 * b * h * d * (s * (s + 1) / 2.0)      # the causal mask leaves S (S + 1) / 2 scores per head
        dense_tf = flops / (ms * 1e-3) / 1e12
        useful_tf = useful / (ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"] if amp else peaks["bf16_tflops"] / 2.0 / 3.0
        nominal = NOMINAL["bf16_tflops"] if amp else NOMINAL["bf16_tflops"] / 2.0 / 3.0
        out["attention"].append({"workload": f"causal SDPA B={b} H={h} S={s} D={d} {'bf16 autocast' if amp else 'fp32 (3xTF32)'}, additive mask",
                                 "tokens_per_s": b * s / (ms * 1e-3), "plan_ms": ms, "kernel_ms": k_ms, "kernels": trace,
                                 "dense_equivalent_tflops": dense_tf, "causal_useful_tflops": useful_tf,
                                 "roofline": {"bound": "tensor", "achieved": dense_tf, "peak": peak, "unit": "TFLOP/s",
                                              "frac": dense_tf / peak, "useful_achieved": useful_tf, "useful_frac": useful_tf / peak,
                                              "frac_of_nominal": dense_tf / nominal, "useful_frac_of_nominal": useful_tf / nominal,
                                              "basis": "plan time (operand staging included); dense-equivalent counts the masked "
                                                       "half of the score matrix as if computed, useful counts S(S+1)/2 scores per head",
                                              "peak_note": "measured cuBLAS bf16 burst" if amp else
                                              "measured bf16 burst / 2 (tf32) / 3 (three products per result)"}})
        del arrays, store, t
    if "gemm_widths" in want:
        # the decoder's projection shapes with the CTA-pair tile width forced (0 = the launcher's own choice)
        out["gemm_widths"] = []
        for (m, n, k) in ((8192, 768, 768), (8192, 768, 3072), (8192, 3072, 768), (8192, 2304, 768), (4096, 4096, 4096)):
            for amp in ("", "bfloat16"):
                arrays = configs.linear_inputs(m, n, k)
                store = graph.BufferStore()
                t = {kk: graph.from_numpy(v, store) for kk, v in arrays.items()}
                root = configs.linear_gelu(graph, t, amp)
                row = {"workload": f"Linear+bias+GELU M={m} N={n} K={k} {'bf16 autocast' if amp else 'fp32 (3xTF32)'}", "us_per_launch": {}}
                for width in (256, 192, 128, 0):
                    bridge.set_option("gemm_pair_tile_width", width)
                    ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, max(5, steps // 4))
                    gemm = [p for p in prof if p["name"].startswith("gemm")]
                    row["us_per_launch"]["auto" if width == 0 else str(width)] = 1e3 * gemm[0]["ms"] / max(gemm[0]["launches"], 1)
                out["gemm_widths"].append(row)
                del arrays, store, t
    if "gpt" in want:
        arrays = configs.gpt_inputs(batch=8)
        meta = arrays.pop("_meta")
        store = graph.BufferStore()
        t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
        gpt_steps = max(3, steps // 2)
        # the fp32 graph (contractions on the 3xTF32 path), then the same decoder built under autocast: float16 is the
        # dtype the reference's AMP pass pins, bfloat16 follows the same cast rule
        for amp, label in (("", "fp32 graph (3xTF32)"), ("float16", "float16 autocast"), ("bfloat16", "bfloat16 autocast")):
            root = configs.gpt_forward(graph, t, meta, amp=amp)
            ms, prof, trace = time_plan(bridge, torch, stream, root, store, front, gpt_steps)
            top = sorted(prof, key=lambda p: -p["ms"])[:6]
            out["gpt"].append({"workload": f"GPT decoder forward 12L d768 h12 mlp3072 V32000 seq1024, batch 8 (one GPU's shard of 64), {label}",
                               "tokens_per_s": 8 * 1024 / (ms * 1e-3), "plan_ms": ms, "units": len(trace),
                               "top_kernels": [{"name": p["name"], "ms_per_forward": p["ms"] / p["runs"]} for p in top]})
        del arrays, store, t
    return out


def collective_extras(bridge, torch, dist, world: int, rank: int, local: int, reps: int = 5) -> dict:
    """The data-path collectives of configuration 5 (GPT decoder, batch 64 split 8 per GPU) at N > 1, wall-clock
    between two barriers, slowest of the ranks: (i) the hidden states of every rank's shard all-gathered on the devices
    ([8192, 768] fp32 per rank) and (ii) the LM head ([32000, 768]) split along its output columns, each rank
    multiplying the gathered hidden states by its own block, the logits blocks all-gathered and laid side by side.
    Hidden states and weights are seeded synthetic values of the configuration's shapes (the cost of the exchange does
    not depend on them).  `nccl_all_gather` is a plain all_gather_into_tensor of the same bytes between torch buffers,
    measured in the same run, as the yardstick."""
    from browsergrad_b200 import front, graph, sharded

    def timed(fn) -> float:
        best = None
        for i in range(reps + 1):       # pass 0 warms up (communicator set-up, plan compilation) and is not counted
            dist.barrier()
            bridge.synchronize()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            bridge.synchronize()
            torch.cuda.synchronize()
            dist.barrier()
            dt = time.perf_counter() - t0
            if i > 0:
                best = dt if best is None else min(best, dt)
        t = torch.tensor([best], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows, d_model, vocab = 8 * 1024, 768, 32000
    rng = np.random.default_rng(400 + rank)
    hidden = rng.standard_normal((rows, d_model), dtype=np.float32)
    h_local = bridge.upload(hidden, hidden.shape, "float32")
    out = {}
    # (i) hidden states
    gathered = []

    def gather_hidden():
        while gathered:
            bridge.release(gathered.pop())
        gathered.append(sharded.gather_rows_device(bridge, h_local, (rows, d_model), "float32", world * rows, device=local))
    t_gather = timed(gather_hidden)
    nbytes = world * rows * d_model * 4
    recv = (world - 1) * rows * d_model * 4
    a = torch.empty(rows * d_model, dtype=torch.float32, device=f"cuda:{local}")
    full = torch.empty(world * rows * d_model, dtype=torch.float32, device=f"cuda:{local}")
    t_nccl = timed(lambda: dist.all_gather_into_tensor(full, a))
    out["hidden_gather"] = {"workload": f"all-gather of [{rows},{d_model}] fp32 hidden states per rank into [{world * rows},{d_model}] on every rank",
                            "ms": 1e3 * t_gather, "bytes_received_per_rank": recv, "gbs_per_rank": recv / t_gather / 1e9,
                            "bus_gbs": nbytes * (world - 1) / world / t_gather / 1e9,
                            "nccl_all_gather": {"ms": 1e3 * t_nccl, "gbs_per_rank": recv / t_nccl / 1e9},
                            "frac_of_nccl": t_nccl / t_gather}
    # (ii) column-split LM head on the gathered hidden states
    w = np.random.default_rng(401).standard_normal((vocab, d_model), dtype=np.float32) * np.float32(0.02)
    store = graph.BufferStore()
    table = front.resident_table(bridge) or front.DeviceBufferTable(bridge)
    bridge._front_table = table
    bid = "gathered_hidden"
    table.register(bid, gathered.pop())
    buf = graph.Node("BUFFER", (), (world * rows, d_model), "float32", bid)
    x = graph.Tensor(graph.Node("LOAD", (buf,), buf.shape, buf.dtype, None), front._ResidentStore(store, table, bridge))
    results = []
    w_block = sharded.weight_block(w, x._store)       # this rank's [vocab / world, d_model] rows: uploaded by the first call, resident after

    def lm_head():
        while results:
            t_out = results.pop()
            table.release(t_out._uop.inputs[0].arg)
        results.append(sharded.column_split_linear(bridge, x, w_block, None, device=local))
    t_head = timed(lm_head)
    m = world * rows
    logits_bytes = m * vocab * 4
    recv_head = logits_bytes * (world - 1) // world
    a2 = torch.empty(m * (vocab // world), dtype=torch.float32, device=f"cuda:{local}")
    full2 = torch.empty(m * vocab, dtype=torch.float32, device=f"cuda:{local}")
    t_nccl2 = timed(lambda: dist.all_gather_into_tensor(full2, a2))
    del a2, full2
    out["lm_head_column_split"] = {"workload": f"logits [{m},{vocab}] fp32 = hidden [{m},{d_model}] . W^T, W split {vocab // world} columns per rank "
                                               "(3xTF32), blocks all-gathered on the devices and laid side by side",
                                   "ms": 1e3 * t_head, "bytes_received_per_rank": recv_head, "gbs_per_rank": recv_head / t_head / 1e9,
                                   "tflops_per_rank": 2.0 * m * (vocab // world) * d_model / t_head / 1e12,
                                   "nccl_all_gather": {"ms": 1e3 * t_nccl2, "gbs_per_rank": recv_head / t_nccl2 / 1e9},
                                   "all_gather_share_of_time": t_nccl2 / t_head}
    while results:
        t_out = results.pop()
        table.release(t_out._uop.inputs[0].arg)
    table.release(bid)
    bridge.release(h_local)
    return out


def bind_to_gpu_numa_node(torch, local: int):
    """Restrict this process to the cores of the NUMA node the GPU hangs off (read from sysfs), so that page-locked
    buffers allocated from now on are first touched there.  Returns (previous affinity or None, a description)."""
    try:
        prop = torch.cuda.get_device_properties(local)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as fh:
            node = int(fh.read().strip())
        if node < 0:
            return None, {"node": None, "note": "the platform reports no NUMA node for the GPU"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        old = os.sched_getaffinity(0)
        usable = cpus & old
        if not usable:
            return None, {"node": node, "note": "none of the node's cores is available to this process"}
        os.sched_setaffinity(0, usable)
        return old, {"node": node, "cores": len(usable)}
    except Exception as exc:      # no sysfs, no permission: run unbound
        return None, {"node": None, "note": repr(exc)}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_rows = 1024
    kind, _ = cpu_reference_realize()
    workers = os.cpu_count() or 1
    per_step = cpu_reference_steps(sample_rows, workers, max(1, args.warmup), args.steps)
    total = sum(per_step)
    nbytes = workers * sum(algorithmic_bytes(sample_rows, COLS).values())
    value = nbytes * args.steps / total / 1e9
    sample = (f"{workers} processes x {sample_rows} of {ROWS} rows x {COLS} cols per step (NumPy runs this path on one "
              f"thread per process), NumPy {np.__version__}")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_step": workers * sample_rows, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": workers, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="cuda")
    ap.add_argument("--rows", type=int, default=ROWS)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--only", default="", help="comma-separated extra workloads to run instead of the main benchmark: "
                    + ", ".join(EXTRA_NAMES))
    ap.add_argument("--attn-batch", type=int, default=16)
    ap.add_argument("--extra-warmup", type=int, default=3, help="untimed realizations before each --only workload")
    ap.add_argument("--e2e-chunks", type=int, default=16)
    ap.add_argument("--e2e-lanes", type=int, default=4)
    ap.add_argument("--option", action="append", default=[], metavar="KEY=VALUE",
                    help="bridge option set before anything runs (repeatable), e.g. attention16_kernel=3")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from browsergrad_b200 import CudaBridge, configs, front, graph, realize_cuda

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a rank that fails must not leave the others waiting for the default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=240))
    rows = args.rows
    bytes_step = algorithmic_bytes(rows, COLS)
    total_bytes = sum(bytes_step.values())

    bridge = CudaBridge(local)
    for kv in args.option:
        key, _, val = kv.partition("=")
        bridge.set_option(key, int(val))
    stream = torch.cuda.ExternalStream(bridge.stream(), device=local)
    if args.only:
        global EXTRA_WARMUP
        EXTRA_WARMUP = max(0, args.extra_warmup)
        names = [n for n in args.only.split(",") if n]
        bad = [n for n in names if n not in EXTRA_NAMES + ("gemm_widths",)]
        if bad:
            raise SystemExit(f"unknown workload(s) {bad}; choose from {EXTRA_NAMES + ('gemm_widths',)}")
        res = extra_measurements(bridge, torch, stream, measured_peaks(), max(1, args.steps), names, args.attn_batch)
        if rank == 0:
            print(json.dumps({"only": names, "extra": res}))
        bridge.close()
        return
    arrays = configs.chain_inputs(rows, COLS)   # every rank: its own shard of the same size (weak scaling)
    if world > 1:
        for k in arrays:  # distinct data per rank
            arrays[k] = np.roll(arrays[k], rank, axis=0)
    store, t, roots = build_graphs(graph, configs, arrays)
    table = front.DeviceBufferTable(bridge)
    plans = {}
    for name, root in roots.items():
        prepared, plan = front.plan_for(root._uop)
        inputs = front._bind_inputs(plan, store, table, True)   # uploads the leaves once
        plans[name] = (plan, inputs, prepared.dtype)

    def step() -> None:
        for name in ("y", "rowsum", "rowsoftmax"):
            plan, inputs, dtype = plans[name]
            h = bridge.run_tensor_plan_resident(plan, inputs, dtype)
            bridge.release(h)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        bridge.synchronize()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    bridge.synchronize()
    bridge.flushProfiles()
    bridge.set_option("profiling", 1)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = bridge.resourceSnapshot()["kernelLaunches"]
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = bridge.resourceSnapshot()["kernelLaunches"] - launches0
    clocks = sampler.stop() if rank == 0 else None
    profiles = bridge.flushProfiles()
    bridge.set_option("profiling", 0)
    if world > 1:
        tms = torch.tensor([ms], device=f"cuda:{local}")
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    value = world * total_bytes * args.steps / (ms * 1e-3) / 1e9

    # roofline of the dominant kernel, from the CUDA events recorded around each launch above
    peaks = measured_peaks()
    per_kernel = {}
    for p in profiles:
        key = "rowsoftmax" if "FUSED_SOFTMAX" in p["name"] else ("rowsum" if "REDUCE" in p["name"] else "y")
        per_kernel[key] = {"name": p["name"], "ms": p["ms"] / max(p["launches"], 1), "launches": p["launches"]}
    roofline = None
    if per_kernel:
        top = max(per_kernel, key=lambda k: per_kernel[k]["ms"])
        achieved = bytes_step[top] / (per_kernel[top]["ms"] * 1e-3) / 1e9
        # DRAM read+write per launch: one ncu capture of a smaller case, kept as a tracked file that names the capture,
        # scaled by the rows processed (traffic grows in proportion); the capture understates the write side (see its
        # note), so the figure is floored at the algorithmic bytes
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "config2_pattern_kernels_traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as fh:
                cap = json.load(fh)
            traffic = max(float(cap["bytes_per_launch"][top]) * rows / float(cap["rows"]), float(bytes_step[top]))
        roofline = {"bound": "hbm", "kernel": per_kernel[top]["name"], "achieved": achieved, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                    "frac_of_nominal": achieved / NOMINAL["hbm_gbs"], "nominal_peak": NOMINAL["hbm_gbs"],
                    "traffic": traffic, "traffic_source": "profiles/config2_pattern_kernels_traffic.json (scaled by rows, floored at the algorithmic bytes)",
                    "algorithmic_bytes": bytes_step[top],
                    "per_kernel": {k: {"name": v["name"], "ms_per_launch": v["ms"],
                                       "achieved_gbs": bytes_step[k] / (v["ms"] * 1e-3) / 1e9,
                                       "frac": bytes_step[k] / (v["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"]}
                                   for k, v in per_kernel.items()}}

    # end to end: pinned host inputs -> device -> kernels -> host result, through realize_cuda
    e2e = None
    if not args.no_e2e:
        # host threads and the page-locked buffers they first touch go to the NUMA node of this rank's GPU for the
        # length of this section (the CPU baseline below gets all cores back)
        old_affinity, numa = bind_to_gpu_numa_node(torch, local)
        # one step = host inputs -> device (once per step, shared by the three realizations), three
        # realizations, each result read back into page-locked host memory; leaves are dropped at step end
        from browsergrad_b200 import release_resident_leaves
        pinned = {k: torch.from_numpy(v).pin_memory().numpy() for k, v in arrays.items()}
        pstore, pt, proots = build_graphs(graph, configs, pinned)
        outs = {"y": torch.empty((rows, COLS), dtype=torch.float32).pin_memory().numpy(),
                "rowsum": torch.empty((rows,), dtype=torch.float32).pin_memory().numpy(),
                "rowsoftmax": torch.empty((rows, COLS), dtype=torch.float32).pin_memory().numpy()}
        h2d = sum(v.nbytes for v in pinned.values())
        d2h = sum(v.nbytes for v in outs.values())

        def e2e_step() -> None:
            for name in ("y", "rowsum", "rowsoftmax"):
                realize_cuda(proots[name], bridge, resident_leaves=True, out=outs[name])
            release_resident_leaves(bridge)

        def timed(fn, n: int) -> float:
            fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            barrier()
            dt = time.perf_counter() - t0
            if world > 1:
                tdt = torch.tensor([dt], device=f"cuda:{local}")
                dist.all_reduce(tdt, op=dist.ReduceOp.MAX)
                dt = float(tdt.item())
            return dt
        n_e2e = max(2, min(args.steps, 10))
        dt_single = timed(e2e_step, n_e2e)
        # the same step streamed in row chunks over several bridges (one stream each) of this device, so that
        # uploads, kernels and read-backs of neighbouring chunks overlap on the full-duplex PCIe link
        from browsergrad_b200.sharded import cuda_row_pipeline
        lanes = [bridge] + [CudaBridge(local) for _ in range(max(1, args.e2e_lanes) - 1)]
        pipe = cuda_row_pipeline(lambda tt: {"y": configs.chain_y(graph, tt), "rowsum": configs.chain_rowsum(graph, tt),
                                             "rowsoftmax": configs.chain_rowsoftmax(graph, tt)},
                                 pinned, list(pinned), lanes, n_chunks=args.e2e_chunks)
        dt = timed(lambda: pipe.run(outs), n_e2e)
        for extra_bridge in lanes[1:]:
            extra_bridge.close()
        # the ceiling the link sets: the same bytes copied with bare asynchronous copies between the same page-locked
        # buffers and device memory, uploads and read-backs on two streams at once, no kernels; all ranks at the same time
        dev_in = {k: torch.empty(v.shape, dtype=torch.float32, device=f"cuda:{local}") for k, v in pinned.items()}
        dev_out = {k: torch.empty(v.shape, dtype=torch.float32, device=f"cuda:{local}") for k, v in outs.items()}
        pin_in = {k: torch.from_numpy(v) for k, v in pinned.items()}
        pin_out = {k: torch.from_numpy(v) for k, v in outs.items()}
        s_up, s_down = torch.cuda.Stream(device=local), torch.cuda.Stream(device=local)

        def bare_copies() -> None:
            with torch.cuda.stream(s_up):
                for k in dev_in:
                    dev_in[k].copy_(pin_in[k], non_blocking=True)
            with torch.cuda.stream(s_down):
                for k in dev_out:
                    pin_out[k].copy_(dev_out[k], non_blocking=True)
            s_up.synchronize()
            s_down.synchronize()
        dt_copy = timed(bare_copies, n_e2e)
        del dev_in, dev_out
        if old_affinity is not None:
            os.sched_setaffinity(0, old_affinity)
        e2e = {"value": world * total_bytes * n_e2e / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
               "copy_ceiling": {"value": world * total_bytes * n_e2e / dt_copy / 1e9, "ms_per_step": 1e3 * dt_copy / n_e2e,
                                "what": "bare cudaMemcpyAsync of the same bytes, both directions at once, no kernels, all ranks together",
                                "e2e_over_ceiling": dt_copy / dt},
               "numa": numa,
               "d2h_bytes_per_step": d2h, "steps": n_e2e, "ms_per_step": 1e3 * dt / n_e2e,
               "api": f"sharded.cuda_row_pipeline(...).run(outs): {args.e2e_chunks} row chunks over {len(lanes)} bridges",
               "single_call": {"value": world * total_bytes * n_e2e / dt_single / 1e9, "ms_per_step": 1e3 * dt_single / n_e2e,
                               "api": "realize_cuda(root, out=pinned) per root, leaves uploaded once per step"}}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(1024, repeats=2)
    extra = None
    if rank == 0 and world == 1 and not args.no_extra:
        table.release_all()
        try:
            extra = extra_measurements(bridge, torch, stream, peaks, max(3, min(args.steps, 10)))
        except Exception as exc:   # the headline line must survive a failure in the extras
            extra = {"error": repr(exc)}
    elif world > 1 and not args.no_extra:
        # the batch-sharded configurations on every rank (its own shard of the same size): one GPU's shard of the
        # GPT decoder, the causal attention config and the largest bf16 Linear; aggregate = N x work / slowest rank
        table.release_all()
        mine, failure, vals = None, None, [float("nan")] * 4
        try:
            mine = extra_measurements(bridge, torch, stream, peaks, max(3, min(args.steps, 10)),
                                      ("gpt", "attn_bf16", "attn_fp32", "gemm_bf16_8192"), args.attn_batch)
            vals = [mine["gpt"][0]["plan_ms"], mine["attention"][0]["plan_ms"], mine["attention"][1]["plan_ms"],
                    mine["gemm"][0]["plan_ms"]]
        except Exception as exc:   # every rank still joins the reduction below
            failure = repr(exc)
        times = torch.tensor(vals, device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)     # NaN from a failed rank propagates
        gpt_ms, attn32_ms, attn16_ms, gemm_ms = (float(x) for x in times.tolist())
        if mine is None or any(x != x for x in (gpt_ms, attn32_ms, attn16_ms, gemm_ms)):
            extra = {"error": failure or "a rank failed its sharded extras"}
        else:
            extra = {"note": f"every rank runs its own shard; times are the slowest rank's, throughput is the sum over {world} ranks",
                     "gpt": {"workload": mine["gpt"][0]["workload"], "ms_per_forward": gpt_ms,
                             "tokens_per_s": world * 8 * 1024 / (gpt_ms * 1e-3)},
                     "attention": [{"workload": mine["attention"][0]["workload"], "plan_ms": attn32_ms,
                                    "tokens_per_s": world * args.attn_batch * 2048 / (attn32_ms * 1e-3)},
                                   {"workload": mine["attention"][1]["workload"], "plan_ms": attn16_ms,
                                    "tokens_per_s": world * args.attn_batch * 2048 / (attn16_ms * 1e-3)}],
                     "gemm": {"workload": mine["gemm"][0]["workload"], "plan_ms": gemm_ms,
                              "tflops": world * 2.0 * 8192 ** 3 / (gemm_ms * 1e-3) / 1e12}}
        try:
            coll = collective_extras(bridge, torch, dist, world, rank, local)
            if isinstance(extra, dict):
                extra["collectives"] = coll
        except Exception as exc:       # every rank runs the same calls; a failure is reported, not hidden
            if isinstance(extra, dict):
                extra["collectives"] = {"error": repr(exc)}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_step": world * rows, "rows_per_gpu": rows,
                       "algorithmic_bytes_per_step": total_bytes, "l2": "inputs (4 x 268 MB) exceed the 126 MB L2",
                       "parallelism": f"row-sharded x{world}, no collective"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line))
    table.release_all()
    bridge.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
