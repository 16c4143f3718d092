"""Benchmark of the attention hot path: `python bench.py --gpus N --steps K --warmup W`.

Metric: attention throughput in TFLOP/s (and ms per layer), FLOPs = 4 * L^2 * 128 * H as the
reference counts them (src/bin/mmh3-tools/bench.rs:141). A step is one attention layer over one
batch of seeded synthetic activations.

- N = 1: dense BF16 attention at L = 65,536 + 512 text tokens, H = 32, D = 128 (the configuration the
  metric is quoted on). The same line carries the INT8/FP8 kernel, the fused quantize pass and the
  video-sparse path as extra keys.
- N > 1 (launched by torch.distributed.run, one rank per GPU): the head-sharded (Ulysses) video
  attention layer, L = 124,992 + 512, H = 32, sequence-sharded inputs, NCCL all-to-all both ways,
  dense attention on 32 / N heads per rank. The total work is fixed, so scaling is strong.
- `--impl reference`: the reference's CPU attention path (the f64 oracle restating
  crates/mmh3-cpu/src/dit.rs:79-118; Rust is not installed here) on every host core this process
  may run on, each step a sample of query rows of the same workload sized by time so that the
  whole run ends within a minute or two. Its `ms_per_step` is the time of one sample; the layer
  time extrapolated from it is in `cpu_baseline`. At N = 1 the line's `extra` also carries the
  reference's own CUDA kernels (compiled for sm_100a, oracle/_ref) timed on the same inputs.

Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

REPO = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "tests"))

HEAD_DIM = 128
HEADS = 32
DENSE_TOKENS = 65536 + 512
VIDEO_TOKENS = 124992 + 512
# DRAM bytes per token and head of the dense kernel: 404.7 MB read + 116.2 MB written in the ncu
# capture of one launch at L = 16,384, H = 32 (q, k, v, output once each would be 1,024 B).
DENSE_TRAFFIC_PER_TOKEN = 521.0e6 / (16384 * 32)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def attention_flops(tokens: int, heads: int) -> float:
    return 4.0 * tokens * tokens * HEAD_DIM * heads


def measured_peaks() -> tuple[dict, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) on a thread while
    the timed region runs; nvidia-smi in loop mode stands in where NVML cannot be loaded."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    PERIOD = 0.005

    def __init__(self, index: int):
        self.index = index
        self.process = None
        self.thread = None
        self.stop = threading.Event()
        # (host time, SM MHz, max SM MHz, active reasons)
        self.samples: list[tuple[float, float, float, tuple[str, ...]]] = []
        self.window = (0.0, float("inf"))
        self.source = None

    def _nvml_handle(self):
        import pynvml
        import torch

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(self.index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid)

    def __enter__(self):
        try:
            nvml, handle = self._nvml_handle()
            nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
            self.source = "nvml"
            self.thread = threading.Thread(target=self._poll, args=(nvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.source = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _poll(self, nvml, handle):
        masks = {
            "hw_slowdown": nvml.nvmlClocksThrottleReasonHwSlowdown,
            "hw_thermal_slowdown": nvml.nvmlClocksThrottleReasonHwThermalSlowdown,
            "sw_thermal_slowdown": nvml.nvmlClocksThrottleReasonSwThermalSlowdown,
            "sw_power_cap": nvml.nvmlClocksThrottleReasonSwPowerCap,
        }
        try:
            maximum = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
        except Exception:
            maximum = float("nan")
        while not self.stop.is_set():
            try:
                clock = float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM))
                bits = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                active = tuple(name for name, mask in masks.items() if bits & mask)
                self.samples.append((time.time(), clock, maximum, active))
            except Exception:
                pass
            self.stop.wait(self.PERIOD)

    def _read(self):
        for line in self.process.stdout:
            fields = [field.strip() for field in line.split(",")]
            if len(fields) != 7:
                continue
            try:
                clock, maximum = float(fields[0]), float(fields[1])
            except ValueError:
                continue
            active = tuple(name for name, flag in zip(self.NAMES, fields[3:])
                           if flag.lower().startswith("active"))
            self.samples.append((time.time(), clock, maximum, active))

    def mark(self, start: float, end: float) -> None:
        """Only samples taken between `start` and `end` (host clock) count."""
        self.window = (start, end)

    def __exit__(self, *_):
        self.stop.set()
        if self.process is not None:
            self.process.terminate()
            self.process.wait(timeout=5)
        if self.thread is not None:
            self.thread.join(timeout=5)

    def summary(self) -> dict:
        inside = [sample for sample in self.samples
                  if self.window[0] <= sample[0] <= self.window[1]]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0,
                    "source": self.source}
        reasons = sorted({name for sample in inside for name in sample[3]})
        return {"sm_mhz": statistics.median(sample[1] for sample in inside),
                "sm_max_mhz": max(sample[2] for sample in inside),
                "reasons": reasons, "samples": len(inside), "source": self.source}


def host_cores() -> int:
    """The cores this process may run on. torch.distributed.run exports OMP_NUM_THREADS=1 to its
    ranks, so OpenMP's own default is not the core count there; the affinity mask is."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_attention_sampler(tokens: int, heads: int, seed: int, qkv=None, threads: int = 0):
    """A function sample(rows, threads=None) that times the CPU oracle on `rows` query rows of
    every head against all keys of the workload and returns (seconds, flops, threads used)."""
    import numpy as np
    import torch

    import oracle_lib
    from mmh3_b200 import synthetic

    oracle = oracle_lib.load()
    cores = threads or host_cores()
    if qkv is None:
        qkv = synthetic.dense_qkv(tokens, heads, seed)
    bits = qkv.view(torch.int16).numpy().view(np.uint16)
    first = (tokens // 2 // 64) * 64

    def sample(rows: int, threads: int | None = None):
        used = threads or cores
        start = time.perf_counter()
        oracle_lib.attention_bf16(oracle, bits, tokens, heads, synthetic.softmax_scale(), first,
                                  first + rows, 0, heads, used)
        seconds = time.perf_counter() - start
        return seconds, 4.0 * rows * tokens * HEAD_DIM * heads, used

    return sample


def workload_config(gpus: int, tokens: int, heads: int) -> dict:
    """What both arms say about the workload, key for key."""
    config = {"workload": workload_name(gpus), "tokens": tokens, "heads": heads,
              "head_dim": HEAD_DIM, "flops_per_step": attention_flops(tokens, heads),
              "l2": f"inputs ({tokens * 3 * heads * HEAD_DIM * 2 / 1e9:.2f} GB) exceed L2 (126 MB)"}
    if gpus > 1:
        config["parallelism"] = f"ulysses{gpus}"
    return config


def run_reference(args) -> None:
    """The reference arm: the CPU path on the box's host cores, rank 0 only. A step is a sample of
    query rows; the row count is chosen once, from a short calibration, so that warm-up and steps
    together take about a minute whatever the core count."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    tokens = DENSE_TOKENS if args.gpus == 1 else VIDEO_TOKENS
    sample = cpu_attention_sampler(tokens, HEADS, 1)
    seconds, flops, used = sample(2)
    per_row = seconds / 2
    budget = min(2.5, args.reference_seconds / max(1, args.warmup + args.steps))
    rows = max(1, min(args.cpu_rows, int(budget / per_row)))
    times = []
    for step in range(args.warmup + args.steps):
        seconds, flops, used = sample(rows)
        if step >= args.warmup:
            times.append(seconds)
    mean = sum(times) / len(times)
    value = flops / mean / 1e12
    layer_flops = attention_flops(tokens, HEADS)
    described = (f"{rows} query rows x {HEADS} heads against all {tokens} keys per step "
                 f"({flops / 1e9:.1f} GFLOP of the layer's {layer_flops / 1e12:.1f} TFLOP, "
                 f"{mean:.2f} s; a whole layer at this rate would take "
                 f"{mean * layer_flops / flops:.0f} s)")
    line = {
        "impl": "reference", "metric": "attention_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": workload_config(args.gpus, tokens, HEADS),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": used, "kind": "port",
                         "sample": described},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "step_is": "a sample of query rows of the layer, not a whole layer",
        # What `value` times: the reference's CPU path. Its CUDA kernels on the same rows are
        # under extra.reference_cuda_kernels at N = 1.
        "reference_class": "cpu",
    }
    if args.gpus == 1 and not args.no_reference_kernels:
        line["extra"] = {"reference_cuda_kernels": reference_kernel_times(tokens, HEADS)}
    print(json.dumps(line))


def reference_kernel_times(tokens: int, heads: int, qkv=None, output=None) -> dict:
    """The reference's own CUDA kernels for the path (its mma.sync / cp.async code compiled
    unchanged for sm_100a into oracle/_ref) on the benchmark's inputs on this GPU: dense BF16, and
    INT8/FP8 over a workspace it prepared itself. They run on the legacy default stream, outside
    every timed region of this library's kernels; none of this library's kernels run here."""
    try:
        import torch

        import oracle_lib
        from mmh3_b200 import _lib, synthetic

        reference = oracle_lib.load_reference()
        if reference is None or not torch.cuda.is_available():
            return {"unavailable": "oracle/_ref/libmmh3_ref.so is not built or no GPU is visible"}
        torch.cuda.set_device(0)
        inner = heads * HEAD_DIM
        scale = synthetic.softmax_scale()
        if qkv is None:
            qkv = synthetic.dense_qkv(tokens, heads, seed=1).cuda()
        if output is None:
            output = torch.zeros((tokens, heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
        base = qkv.data_ptr()
        flops = attention_flops(tokens, heads)

        def dense():
            code = reference.mmh3_attention_bf16(base, base + 2 * inner, base + 4 * inner,
                                                 output.data_ptr(), tokens, heads, 3 * inner,
                                                 3 * inner, 3 * inner, inner, scale, None)
            if code != 0:
                raise RuntimeError(f"the reference's mmh3_attention_bf16 returned {code}")

        torch.cuda.synchronize()
        dense()
        ms = time_region(torch, dense, 2)
        result = {"dense_bf16": {"ms": ms, "tflops": flops / ms / 1e9},
                  "library": "oracle/_ref/libmmh3_ref.so (the reference's kernels, sm_100a)",
                  "stream": "legacy default"}
        blocks = -(-tokens // 64)
        byte = dict(dtype=torch.uint8, device="cuda")
        real = dict(dtype=torch.float32, device="cuda")
        buffers = [torch.empty(tokens * inner, **byte), torch.empty(tokens * inner, **byte),
                   torch.empty(blocks * 64 * inner, **byte), torch.empty(heads * blocks, **real),
                   torch.empty(heads * blocks, **real), torch.empty(heads, **real),
                   torch.empty(heads * blocks, **real)]
        workspace = _lib.QuantizedWorkspaceStruct(*(buffer.data_ptr() for buffer in buffers))
        layout = _lib.AttentionLayout()
        for index in range(4):
            layout.token_stride[index] = inner if index == 3 else 3 * inner
            layout.head_stride[index] = HEAD_DIM

        def quantized(ready):
            code = reference.mmh3_attention_quantized(
                base, base + 2 * inner, base + 4 * inner, output.data_ptr(), tokens, heads,
                ctypes.byref(layout), scale, None, ctypes.byref(workspace), ready, None)
            if code != 0:
                raise RuntimeError(f"the reference's mmh3_attention_quantized returned {code}")

        quantized(0)
        ms = time_region(torch, lambda: quantized(2), 2)
        result["int8_fp8_prepared"] = {"ms": ms, "tflops": flops / ms / 1e9}
        return result
    except Exception as error:  # context only: never a reason to lose the line
        return {"unavailable": str(error)[:160]}


def eight_bit_peaks(torch) -> dict:
    """INT8 and FP8 GEMM rates of this GPU from the vendor library, measured the way the BF16 peak
    in MEASURED_PEAKS.json is: 8192^3, best of 10 after a warm-up, CUDA events. They anchor the
    roofline fractions of the INT8/FP8 attention and of the INT8 projection."""
    size = 8192
    operations = 2.0 * size ** 3
    result = {"how": f"{size}^3, best of 10, CUDA events; torch._int_mm and torch._scaled_mm"}

    def best(call):
        call()
        torch.cuda.synchronize()
        fastest = float("inf")
        for _ in range(10):
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record()
            call()
            end.record()
            torch.cuda.synchronize()
            fastest = min(fastest, start.elapsed_time(end))
        return operations / fastest / 1e9

    try:
        a = torch.randint(-127, 128, (size, size), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 128, (size, size), dtype=torch.int8, device="cuda").t()
        result["int8_tops"] = best(lambda: torch._int_mm(a, b))
    except Exception as error:
        result["int8_error"] = str(error)[:120]
    try:
        a = torch.randn((size, size), device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn((size, size), device="cuda").to(torch.float8_e4m3fn).t()
        one = torch.ones((), device="cuda")
        result["fp8_tflops"] = best(lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one,
                                                             out_dtype=torch.bfloat16))
    except Exception as error:
        result["fp8_error"] = str(error)[:120]
    return result


def workload_name(gpus: int, video: bool = False) -> str:
    if gpus == 1 and video:
        return ("dense BF16 video attention layer, L=124992+512, H=32, D=128, one GPU (the "
                "sharded workload unsharded)")
    if gpus == 1:
        return "dense BF16 attention, L=65536+512, H=32, D=128 (BASELINE configs[1])"
    return (f"Ulysses head-sharded dense BF16 video attention layer, L=124992+512, H=32, D=128, "
            f"{gpus} ranks (BASELINE configs[4])")


def time_region(torch, stream_fn, steps: int, barrier=None, sampler=None) -> float:
    """Milliseconds per step of `stream_fn` over `steps` calls, CUDA events on the current stream,
    synchronized on both sides."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    began = time.time()
    start.record()
    for _ in range(steps):
        stream_fn()
    end.record()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.mark(began, time.time())
    return start.elapsed_time(end) / steps


def run_single(args) -> None:
    import torch

    from mmh3_b200 import attention, synthetic

    torch.cuda.set_device(0)
    tokens, heads = args.tokens or DENSE_TOKENS, args.heads or HEADS
    scale = synthetic.softmax_scale()
    flops = attention_flops(tokens, heads)
    host_qkv = synthetic.dense_qkv(tokens, heads, seed=1, pinned=True)
    qkv = host_qkv.cuda()
    output = torch.zeros((tokens, heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    host_output = torch.empty((tokens, heads, HEAD_DIM), dtype=torch.bfloat16, pin_memory=True)

    def dense():
        attention.dense_bf16(qkv, output, tokens, heads, scale)

    pipeline = attention.HostPipeline(tokens, heads, groups=args.e2e_groups)

    def end_to_end():
        # Host buffers in, host buffers out, through the C ABI call the reference's wrapper makes,
        # a group of heads at a time so that the copies of one group hide behind the attention of
        # another. Every byte of q, k and v crosses the bus every step, and every byte of the
        # output comes back.
        pipeline.run(host_qkv, qkv, output, host_output, scale)

    # The sampler starts before the warm-up (nvidia-smi takes a moment to deliver its first line);
    # only what it reads during the timed steps is kept.
    with ClockSampler(0) as sampler:
        for _ in range(args.warmup):
            dense()
        status = attention.take_status()
        dense_ms = time_region(torch, dense, args.steps, sampler=sampler)
        time.sleep(0.2)
    clocks = sampler.summary()
    for _ in range(max(1, args.warmup // 2)):
        end_to_end()
    e2e_ms = time_region(torch, end_to_end, args.steps)
    status = status or attention.take_status()

    extras = {}
    launches = args.steps
    if not args.dense_only:
        extras = run_extras(torch, attention, synthetic, qkv, output, tokens, heads, scale, args)

    peaks, source = measured_peaks()
    achieved = flops / dense_ms / 1e9
    peak = peaks["bf16_tflops"]
    config = workload_config(1, tokens, heads)
    if (tokens, heads) != (DENSE_TOKENS, HEADS):
        config["workload"] = (f"dense BF16 attention, reduced case L={tokens}, H={heads} (not the "
                              "benchmark configuration)")
    cpu = None
    if not args.no_cpu:
        sample = cpu_attention_sampler(tokens, heads, 1, qkv=host_qkv)
        seconds, sample_flops, used = sample(args.cpu_rows)
        # The reference's attention() is single-threaded: the same loop on one core, on a sample
        # a sixteenth the size.
        single_rows = max(1, args.cpu_rows // 16)
        single_seconds, single_flops, _ = sample(single_rows, threads=1)
        cpu = {"value": sample_flops / seconds / 1e12, "unit": "TFLOP/s", "cores": used,
               "kind": "port",
               "sample": (f"{args.cpu_rows} query rows x {heads} heads against all {tokens} keys "
                          f"({sample_flops / 1e9:.1f} GFLOP, {seconds:.1f} s)"),
               "one_core": {"value": single_flops / single_seconds / 1e12, "unit": "TFLOP/s",
                            "cores": 1,
                            "sample": (f"{single_rows} query rows x {heads} heads against all "
                                       f"{tokens} keys ({single_flops / 1e9:.1f} GFLOP, "
                                       f"{single_seconds:.1f} s): the reference's loop as it "
                                       "runs it, on one thread")}}
    line = {
        "metric": "attention_tflops", "value": achieved, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dense_ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": config,
        "kernel_status": status,
        "e2e": {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": host_qkv.numel() * 2,
                "d2h_bytes_per_step": host_output.numel() * 2,
                "launches_per_step": len(pipeline.groups)},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": DENSE_TRAFFIC_PER_TOKEN * tokens * heads,
                     "traffic_unit": "bytes per launch (dram read + write), scaled in proportion "
                                     "to L x H from the ncu capture at L=16384, H=32 (521.0 MB "
                                     "against 536.9 MB algorithmic)",
                     "algorithmic_bytes": 8.0 * tokens * heads * HEAD_DIM,
                     "peak_source": f"{source} bf16_tflops (burst)",
                     "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"]},
        "cpu_baseline": cpu,
        "clocks": clocks,
        "extra": extras,
    }
    print(json.dumps(line))


def run_extras(torch, attention, synthetic, qkv, output, tokens, heads, scale, args) -> dict:
    """The other kernels of the path at the same shape, each timed with CUDA events."""
    extras = {}
    peaks, source = measured_peaks()
    flops = attention_flops(tokens, heads)
    steps = max(2, args.steps // 2)
    eight_bit = eight_bit_peaks(torch)
    extras["peaks"] = eight_bit
    if args.skip_quantized:
        workspace = prepared = None
    try:
        if args.skip_quantized:
            raise StopIteration
        workspace = attention.QuantizedWorkspace(tokens, heads)
        generator = torch.Generator(device="cpu").manual_seed(2)
        norm = attention.HeadNorm(
            (torch.rand(HEAD_DIM, generator=generator) + 0.5).bfloat16().cuda(),
            (torch.rand(HEAD_DIM, generator=generator) + 0.5).bfloat16().cuda(),
            ((torch.rand((tokens, 48), generator=generator) - 0.5) * 80.0).cuda(), 48, 1e-6)
        prepared = qkv.clone()
        maxima = prepared[:, 2].float().abs().amax(dim=(0, 2)).contiguous()

        def quantize():
            attention.prepare_inputs(prepared, norm, tokens, heads, quantized=workspace,
                                     value_head_maxima=maxima)

        quantize()
        ms = time_region(torch, quantize, steps)
        moved = 3.0 * tokens * heads * HEAD_DIM * 3  # 2 bytes read + 1 byte written per element
        extras["fused_quantize"] = {
            "ms": ms, "gbs": moved / ms / 1e6, "algorithmic_bytes": moved,
            "frac_of_hbm": moved / ms / 1e6 / peaks["hbm_gbs"], "peak_source": source}

        def quantized():
            attention.dense_quantized(prepared, output, scale, workspace,
                                      attention.AttentionInputs.PREPARED_WITH_VALUES)

        quantized()
        ms = time_region(torch, quantized, steps)
        extras["int8_fp8_attention"] = {"ms": ms, "tflops": flops / ms / 1e9}
        # Half the work is INT8, half FP8: the time either peak alone would allow, added up.
        if "int8_tops" in eight_bit and "fp8_tflops" in eight_bit:
            floor_ms = (flops / 2 / eight_bit["int8_tops"] + flops / 2 / eight_bit["fp8_tflops"]) / 1e9
            extras["int8_fp8_attention"]["frac_of_measured_8bit_peaks"] = floor_ms / ms
        extras["kernel_status"] = attention.take_status()
    except StopIteration:
        pass
    except attention.CudaError as error:
        extras["int8_fp8_error"] = str(error)
    del workspace, prepared
    torch.cuda.empty_cache()
    if not args.skip_vsa:
        try:
            extras["vsa"] = run_vsa(torch, attention, synthetic, heads, scale, steps,
                                    args.vsa_frames, args.no_reference_kernels)
        except attention.CudaError as error:
            extras["vsa_error"] = str(error)
    if not args.skip_sol:
        try:
            extras["sol"] = run_sol(torch, attention, qkv, output, tokens, heads, scale, steps)
        except attention.CudaError as error:
            extras["sol_error"] = str(error)
    if not args.skip_gemm:
        try:
            extras["qkv_gemm"] = run_gemm(torch, attention, qkv, tokens, heads, steps)
            if "int8_tops" in eight_bit:
                extras["qkv_gemm"]["frac_of_measured_int8_peak"] = (
                    extras["qkv_gemm"]["tops"] / eight_bit["int8_tops"])
        except attention.CudaError as error:
            extras["qkv_gemm_error"] = str(error)
    if not args.no_reference_kernels:
        extras["reference_kernels"] = reference_kernel_times(tokens, heads, qkv, output)
    if not args.skip_video_layer:
        try:
            extras["video_layer_one_gpu"] = run_video_layer(torch, attention, synthetic, heads,
                                                            scale, steps)
        except attention.CudaError as error:
            extras["video_layer_error"] = str(error)
    return extras


def run_video_layer(torch, attention, synthetic, heads, scale, steps) -> dict:
    """The 125,504-token video layer of the sharded benchmark on this one GPU (the dense kernel
    over all heads, which is what one rank of one runs): the 1-GPU end of the scaling curve,
    measured by the same program that measures the N-GPU end."""
    layout, plan = synthetic.video_plan()
    tokens = len(layout)
    qkv = synthetic.video_qkv_device(layout, plan, heads, seed=3)
    output = torch.zeros((tokens, heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")

    def layer():
        attention.dense_bf16(qkv, output, tokens, heads, scale)

    layer()
    ms = time_region(torch, layer, steps)
    flops = attention_flops(tokens, heads)
    return {"workload": workload_name(1, video=True), "tokens": tokens, "heads": heads, "ms": ms,
            "tflops": flops / ms / 1e9, "kernel_status": attention.take_status()}


def run_gemm(torch, attention, qkv, tokens, heads, steps) -> dict:
    """The step before attention: the INT8 qkv projection [tokens, heads * 128] x
    [3 * heads * 128, heads * 128]^T into the BF16 qkv rows, leaving the per-head maxima of |v|.
    Uniform INT8 operands; the weights (50 MB at 32 heads) stay in L2, the activations stream."""
    from mmh3_b200 import gemm

    inner = heads * HEAD_DIM
    generator = torch.Generator(device="cuda").manual_seed(3)
    activations = torch.randint(-127, 128, (tokens, inner), dtype=torch.int8, device="cuda",
                                generator=generator)
    weights = torch.randint(-127, 128, (3 * inner, inner), dtype=torch.int8, device="cuda",
                            generator=generator)
    activation_scales = torch.rand(tokens, device="cuda", generator=generator) + 0.5
    weight_scales = torch.rand(3 * inner, device="cuda", generator=generator) * 1e-4 + 1e-5
    maxima = torch.zeros(heads, dtype=torch.float32, device="cuda")
    target = torch.empty_like(qkv)

    def project():
        gemm.int8(None, activations, weights, activation_scales, weight_scales,
                  gemm.Output(target.view(torch.int16),
                              column_maxima=gemm.ColumnMaxima(maxima, 2 * inner)),
                  tokens, 3 * inner, inner)

    project()
    ms = time_region(torch, project, steps)
    operations = 2.0 * tokens * 3 * inner * inner
    peaks, source = measured_peaks()
    return {
        "workload": f"qkv projection M={tokens}, N={3 * inner}, K={inner}, INT8 -> BF16 + |v| maxima",
        "ms": ms, "tops": operations / ms / 1e9,
        # No INT8 peak is measured on this pool: twice the measured BF16 rate stands in for it.
        "frac_of_twice_bf16_peak": operations / ms / 1e9 / (2.0 * peaks["bf16_tflops"]),
        "frac_of_twice_bf16_sustained": operations / ms / 1e9 /
        (2.0 * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])),
        "peak_source": source, "kernel_status": attention.take_status(),
    }


def run_sol(torch, attention, qkv, output, tokens, heads, scale, steps) -> dict:
    """Sol-Attn on the dense workload's q, k, v at the reference's default threshold (tau = 1.3),
    with the first 512 tokens (8 blocks) as the always-exact conditioning prefix."""
    workspace = attention.SparseWorkspace(tokens, heads)
    layout = attention.qkv_layout(heads)
    sinks = attention.SparseSinks((0, 8), (0, 0))

    def whole():
        attention.sparse(qkv, output, layout, scale, 1.3, sinks, workspace)

    whole()
    ms = time_region(torch, whole, steps)
    blocks = workspace.blocks
    lengths = torch.full((blocks,), 64.0, dtype=torch.float64, device="cuda")
    lengths[-1] = tokens - (blocks - 1) * 64
    counts = workspace.route_counts.view(heads, blocks).to(torch.int64)
    routes = workspace.routes.view(heads, blocks, blocks)
    routed_keys = torch.zeros((heads, blocks), dtype=torch.float64, device="cuda")
    for head in range(heads):
        mask = torch.arange(blocks, device="cuda")[None, :] < counts[head][:, None]
        entries = ((routes[head].to(torch.int64) & 0xFFFF) * mask).clamp_(0, blocks - 1)
        routed_keys[head] = (lengths[entries] * mask).sum(dim=1)
    sparse_flops = float((routed_keys * lengths[None, :]).sum().item()) * 4.0 * HEAD_DIM
    return {
        "workload": f"Sol-Attn L={tokens}, H={heads}, tau 1.3, 8 prefix blocks exact",
        "ms": ms, "sparse_flops": sparse_flops, "sparse_tflops": sparse_flops / ms / 1e9,
        "dense_equivalent_tflops": attention_flops(tokens, heads) / ms / 1e9,
        "kernel_ms": kernel_times(torch, whole),
        "routed_fraction": workspace.routed_fraction(),
        "kernel_status": attention.take_status(),
    }


def kernel_times(torch, fn) -> dict:
    """Device time of each kernel one call of `fn` launches, by name, from the CUPTI activity
    records torch's profiler collects (milliseconds). Empty when the profiler is unavailable."""
    try:
        from torch.profiler import ProfilerActivity, profile

        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as recorded:
            fn()
            torch.cuda.synchronize()
        times: dict[str, float] = {}
        for event in recorded.events():
            if event.device_time_total > 0:
                name = event.name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
                name = name.split("(")[0].replace("void ", "")
                times[name] = times.get(name, 0.0) + event.device_time_total / 1e3
        return {name: round(ms, 4) for name, ms in times.items()}
    except Exception as error:  # the breakdown is a convenience, never a reason to fail the run
        return {"unavailable": str(error)[:80]}


def reference_vsa_ms(torch, plan, qkv, output, tokens, heads, scale, kept, vsa_layout):
    """The reference's own mmh3_vsa_attention (oracle/_ref, sm_100a) on the same rows, with a
    workspace of its own: milliseconds per layer, or None when that library is not built."""
    try:
        import oracle_lib
        from mmh3_b200 import attention

        reference = oracle_lib.load_reference()
        if reference is None:
            return None
        workspace = attention.VsaWorkspace(plan, tokens, heads)
        raw = workspace.raw()
        inner = heads * HEAD_DIM
        base = qkv.data_ptr()

        def call():
            code = reference.mmh3_vsa_attention(
                base, base + 2 * inner, base + 4 * inner, None, inner, output.data_ptr(), tokens,
                heads, ctypes.byref(vsa_layout), scale, plan.tiles, plan.prefix_tiles, kept,
                ctypes.byref(raw), None, 0, None)
            if code != 0:
                raise RuntimeError(f"the reference's mmh3_vsa_attention returned {code}")

        torch.cuda.synchronize()
        call()
        return time_region(torch, call, 2)
    except Exception:
        return None


def run_vsa(torch, attention, synthetic, heads, scale, steps, frames=31,
            no_reference_kernels=False) -> dict:
    """Video sparse attention on the 31 x 48 x 84 grid + 512 text tokens (BASELINE configs[3]):
    pool, select and token attention timed apart. Inputs are drawn on the device: N(0, 1) plus 0.5 x
    a trilinearly upsampled low-resolution field per head and channel, in the plan's cube order."""
    layout, plan = synthetic.video_plan(frames=frames)
    tokens = len(layout)
    kept = plan.kept_video_tiles(0.875)
    qkv = synthetic.video_qkv_device(layout, plan, heads, seed=3)
    output = torch.zeros((tokens, heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    workspace = attention.VsaWorkspace(plan, tokens, heads)
    vsa_layout = attention.qkv_layout(heads)

    def whole():
        attention.vsa(qkv, None, output, vsa_layout, scale, kept, workspace)

    whole()
    ms = time_region(torch, whole, steps)
    kernels = kernel_times(torch, whole)
    selected = workspace.selected_fraction()
    lengths = torch.tensor(plan.tile_lengths, dtype=torch.float64, device="cuda")
    counts = workspace.route_counts.view(heads, plan.tiles).to(torch.int64)
    # Keys each query tile attends: the sum of the lengths of its routed tiles.
    routed_keys = torch.zeros((heads, plan.tiles), dtype=torch.float64, device="cuda")
    routes = workspace.routes.view(heads, plan.tiles, plan.tiles)
    for head in range(heads):
        # Entries past a row's count are whatever the buffer held: clamp them before they index.
        mask = torch.arange(plan.tiles, device="cuda")[None, :] < counts[head][:, None]
        entries = ((routes[head].to(torch.int64) & 0xFFFF) * mask).clamp_(0, plan.tiles - 1)
        table = lengths[entries]
        routed_keys[head] = (table * mask).sum(dim=1)
    sparse_flops = float((routed_keys * lengths[None, :]).sum().item()) * 4.0 * HEAD_DIM
    # The same layer with the gate of the coarse branch, as VSA-trained checkpoints run it: the
    # selection also leaves softmax(pooled scores) . mean values, which the token attention adds
    # to its rows times the gate.
    gate = torch.randn((tokens, heads * HEAD_DIM), dtype=torch.bfloat16, device="cuda",
                       generator=torch.Generator(device="cuda").manual_seed(4))

    def whole_gated():
        attention.vsa(qkv, gate, output, vsa_layout, scale, kept, workspace)

    whole_gated()
    gated_ms = time_region(torch, whole_gated, steps)
    gated_kernels = kernel_times(torch, whole_gated)
    del gate
    # The same layer in INT8/FP8 over inputs the fused pass prepared (identity norm, no rotation):
    # selection and token attention, as the DiT calls it with inputs_ready = 2.
    del workspace
    quantized = attention.VsaWorkspace(plan, tokens, heads, quantized=True)
    ones = torch.ones(HEAD_DIM, dtype=torch.bfloat16, device="cuda")
    maxima = qkv[:, 2].float().abs().amax(dim=(0, 2)).contiguous()
    attention.prepare_inputs(qkv, attention.HeadNorm(ones, ones, None, 0, 1e-6), tokens, heads,
                             vsa=quantized, value_head_maxima=maxima)

    def whole_quantized():
        attention.vsa(qkv, None, output, vsa_layout, scale, kept, quantized,
                      attention.AttentionInputs.PREPARED_WITH_VALUES)

    whole_quantized()
    quantized_ms = time_region(torch, whole_quantized, steps)
    quantized_kernels = kernel_times(torch, whole_quantized)
    reference_ms = None
    if not no_reference_kernels:
        reference_ms = reference_vsa_ms(torch, plan, qkv, output, tokens, heads, scale, kept,
                                        vsa_layout)
    return {
        "workload": (f"VSA L={tokens} ({plan.prefix_tiles} prefix + {plan.video_tiles} video "
                     f"tiles), H={heads}, kept {kept}"),
        "ms": ms, "sparse_flops": sparse_flops, "sparse_tflops": sparse_flops / ms / 1e9,
        "gated_ms": gated_ms,
        "gated_kernel_ms": gated_kernels,
        "int8_fp8_ms": quantized_ms,
        "int8_fp8_kernel_ms": quantized_kernels,
        "reference_kernels_ms": reference_ms,
        "dense_equivalent_tflops": attention_flops(tokens, heads) / ms / 1e9,
        "kernel_ms": kernels,
        "selected_fraction": selected,
        "expected_selected_fraction": plan.expected_selected_fraction(kept),
        "kernel_status": attention.take_status(),
    }


def run_sharded(args) -> None:
    import torch
    import torch.distributed as dist

    from mmh3_b200 import attention, synthetic
    from mmh3_b200.shard import (HostUlyssesPipeline, OverlappedUlyssesAttention, Shard,
                                 UlyssesAttention)

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    # NCCL's kernels on a high-priority stream: an exchange that runs beside an attention launch
    # takes the next multiprocessors that launch frees instead of waiting for its last block.
    options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=options)
    tokens, heads = VIDEO_TOKENS, HEADS
    scale = synthetic.softmax_scale()
    shard = Shard.even(rank, world, tokens, heads, 1)
    own = shard.own_tokens

    def dense(qkv, output, count, span):
        attention.dense_bf16(qkv, output, count, span, scale)

    layer = UlyssesAttention(shard, tokens, heads, dense, "cuda", torch.bfloat16,
                             pack=attention.shard_pack, unpack=attention.shard_unpack)
    # Every rank draws the whole layer from the same seed (the video configuration's
    # distribution) and keeps its own rows, so the data does not depend on the rank count. Two
    # heads of every token stay on the host for the check against the CPU oracle below.
    video_layout, plan = synthetic.video_plan()
    assert len(video_layout) == tokens
    everything = synthetic.video_qkv_device(video_layout, plan, heads, seed=3)
    checked_heads = sorted({(5 * rank) % heads, heads - 1 - rank % heads})
    checked_qkv = {head: everything[:, :, head:head + 1, :].contiguous().cpu()
                   for head in checked_heads}
    generator_rows = torch.empty((len(own), 3, heads, HEAD_DIM), dtype=torch.bfloat16,
                                 pin_memory=True)
    generator_rows.copy_(everything[own.start:own.stop])
    del everything
    torch.cuda.empty_cache()
    qkv = generator_rows.cuda()
    output = torch.zeros((len(own), heads, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    host_output = torch.empty((len(own), heads, HEAD_DIM), dtype=torch.bfloat16, pin_memory=True)

    # The layer goes through a group of heads at a time (up to four, the first and the last of one
    # head of every rank): on resident inputs so that one group's exchanges hide behind another's
    # attention, end to end so that the copies do too.
    groups = max(1, min(4, len(shard.own_heads)))
    overlapped = OverlappedUlyssesAttention(shard, tokens, heads, dense, groups, "cuda",
                                            torch.bfloat16, pack=attention.shard_pack,
                                            unpack=attention.shard_unpack)

    def step():
        overlapped.run(qkv, output)

    def plain_step():
        layer.run(qkv, output)

    # End to end a group's rows must also cross the bus behind the attention of the group before:
    # a head of every rank does in a quarter of the time its attention takes, less with eight
    # ranks reading the host's memory at once.
    pipeline = HostUlyssesPipeline(shard, tokens, heads, dense, groups,
                                   pack=attention.shard_pack, unpack=attention.shard_unpack,
                                   growth=3.0 if world <= 4 else 1.0)

    def end_to_end():
        pipeline.run(generator_rows, qkv, output, host_output)

    with ClockSampler(local) as sampler:
        for _ in range(args.warmup):
            step()
        ms = time_region(torch, step, args.steps, barrier=dist.barrier, sampler=sampler)
        time.sleep(0.2)
    for _ in range(max(1, args.warmup // 2)):
        end_to_end()
    e2e_ms = time_region(torch, end_to_end, args.steps, barrier=dist.barrier)
    # The same layer with exchange, attention, exchange one after the other over all heads at once:
    # what the overlap buys, and the same bits.
    plain_step()
    plain = output.clone()
    plain_ms = time_region(torch, plain_step, max(2, args.steps // 2), barrier=dist.barrier)
    # The pipelined layer must leave what the layer over resident inputs leaves.
    step()
    resident = output.clone()
    agrees_with_plain = float(torch.equal(resident, plain))
    oracle_error, oracle_rows = sharded_oracle_error(torch, resident, checked_qkv, own, tokens,
                                                     scale)
    end_to_end()
    torch.cuda.synchronize()
    agrees = float(torch.equal(host_output.cuda(), resident)) * agrees_with_plain
    wires = None if args.skip_gemm else sharded_block(torch, dist, attention, args, shard, layer,
                                                      dense, qkv, output, tokens, heads)
    status = attention.take_status()
    times = torch.tensor([ms, e2e_ms, float(status), -agrees, oracle_error, plain_ms],
                         dtype=torch.float64, device="cuda")
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, status, disagrees, oracle_error, plain_ms = times.tolist()
    if rank == 0:
        flops = attention_flops(tokens, heads)
        peaks, source = measured_peaks()
        value = flops / ms / 1e9
        line = {
            "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(world, tokens, heads),
            "kernel_status": int(status),
            "exchange_bytes_per_rank": layer.exchange_bytes(),
            "head_groups": len(overlapped.cuts),
            "without_overlap_ms": plain_ms,
            # Rows of every rank's share of the sharded layer's output against the f64 CPU oracle
            # over all keys of the layer: the largest error over all ranks, and the bound.
            "oracle_check": {"max_abs_error": oracle_error, "bound": 2e-2,
                             "rows_per_rank": oracle_rows, "ranks": world,
                             "passed": oracle_error <= 2e-2},
            "e2e": {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": generator_rows.numel() * 2 * world,
                    "d2h_bytes_per_step": host_output.numel() * 2 * world,
                    "head_groups": len(pipeline.cuts),
                    "equals_resident_run": disagrees == -1.0},
            # per rank, step and group of heads: N packs, the attention kernel, N unpacks (NCCL's
            # kernels aside)
            "gpu_launches": args.steps * (2 * world + 1) * len(overlapped.cuts),
            "roofline": {"bound": "tensor", "achieved": value, "peak": peaks["bf16_tflops"] * world,
                         "unit": "TFLOP/s", "frac": value / (peaks["bf16_tflops"] * world),
                         "traffic": DENSE_TRAFFIC_PER_TOKEN * tokens * heads / world,
                         "traffic_unit": "bytes per rank's launch, scaled from the 1-GPU ncu "
                                         "capture in proportion to L x heads per rank",
                         "peak_source": f"{source} bf16_tflops (burst) x {world}"},
            "cpu_baseline": None,
            "clocks": sampler.summary(),
        }
        if wires is not None:
            line["extra"] = {"projection_and_attention": wires}
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def sharded_oracle_error(torch, output, checked_qkv, own, tokens, scale):
    """The largest difference between rows of this rank's output [own tokens, heads, 128] and the
    f64 CPU oracle over all `tokens` keys, for the first, middle and last of the rank's tokens
    and the heads of `checked_qkv` (head -> BF16 [tokens, 3, 1, 128] on the host). Returns
    (error, rows checked)."""
    import numpy as np

    import oracle_lib

    oracle = oracle_lib.load()
    worst, count = 0.0, 0
    rows = sorted({own.start, own.start + len(own) // 2, own.stop - 1})
    for head, host in checked_qkv.items():
        bits = host.view(torch.int16).numpy().view(np.uint16)
        for row in rows:
            expected = oracle_lib.attention_bf16(oracle, bits, tokens, 1, scale, row, row + 1,
                                                 0, 1, host_cores())
            actual = output[row - own.start, head].float().cpu().numpy()
            worst = max(worst, float(np.max(np.abs(actual - expected[0, 0]))))
            count += 1
    return worst, count


def sharded_block(torch, dist, attention, args, shard, layer, dense, qkv, output, tokens,
                  heads) -> dict:
    """The INT8 qkv projection and the attention of one sharded block, with either wire format:
    q, k and v exchanged after projecting this rank's tokens onto every head (two all-to-alls), or
    the INT8 block input gathered and every token projected onto this rank's heads (an all-gather
    and one all-to-all). Both do the same arithmetic per rank and must give the same bits."""
    from mmh3_b200 import gemm
    from mmh3_b200.shard import ProjectedUlyssesAttention, own_projection_rows

    inner = heads * HEAD_DIM
    own = shard.own_tokens
    generator = torch.Generator(device="cuda").manual_seed(5)
    weights = torch.randint(-127, 128, (3 * inner, inner), dtype=torch.int8, device="cuda",
                            generator=generator)
    weight_scales = torch.rand(3 * inner, device="cuda", generator=generator) * 2e-4 + 1e-4
    generator.manual_seed(7 + own.start)
    rows = torch.randint(-127, 128, (len(own), inner), dtype=torch.int8, device="cuda",
                         generator=generator)
    row_scales = torch.rand(len(own), device="cuda", generator=generator) * 0.02 + 0.01
    selected = own_projection_rows(heads, shard.own_heads).cuda()
    own_weights = weights[selected].contiguous()
    own_weight_scales = weight_scales[selected].contiguous()

    def project_own_heads(part_rows, part_scales, target):
        gemm.int8(None, part_rows, own_weights, part_scales, own_weight_scales,
                  gemm.Output(target.view(torch.int16)), part_rows.shape[0],
                  own_weights.shape[0], inner)

    projected = ProjectedUlyssesAttention(shard, tokens, heads, inner, project_own_heads, dense,
                                          "cuda", torch.bfloat16, unpack=attention.shard_unpack)

    def wire_qkv():
        gemm.int8(None, rows, weights, row_scales, weight_scales,
                  gemm.Output(qkv.view(torch.int16)), len(own), 3 * inner, inner)
        layer.run(qkv, output)

    def wire_rows():
        projected.run(rows, row_scales, output)

    steps = max(2, args.steps // 2)
    wire_qkv()
    first = output.clone()
    qkv_ms = time_region(torch, wire_qkv, steps, barrier=dist.barrier)
    wire_rows()
    agree = float(torch.equal(first, output))
    rows_ms = time_region(torch, wire_rows, steps, barrier=dist.barrier)
    times = torch.tensor([qkv_ms, rows_ms, -agree], dtype=torch.float64, device="cuda")
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    qkv_ms, rows_ms, disagree = times.tolist()
    return {
        "workload": f"INT8 qkv projection (K = {inner}) + dense attention, L={tokens}, H={heads}",
        "qkv_wire_ms": qkv_ms, "qkv_wire_bytes_per_rank": layer.exchange_bytes(),
        "int8_wire_ms": rows_ms, "int8_wire_bytes_per_rank": projected.exchange_bytes(),
        "outputs_identical": disagree == -1.0,
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--cpu-rows", type=int, default=32,
                        help="query rows per head of the CPU baseline's sample")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--tokens", type=int, default=0,
                        help="a reduced sequence length for profiler captures (N = 1 only)")
    parser.add_argument("--heads", type=int, default=0,
                        help="a reduced head count for profiler captures (N = 1 only)")
    parser.add_argument("--skip-sol", action="store_true", help="leave Sol-Attn out")
    parser.add_argument("--e2e-groups", type=int, default=0,
                        help="groups of heads the end-to-end leg pipelines its copies over "
                             "(1: copy in, attend, copy out, one after the other)")
    parser.add_argument("--skip-gemm", action="store_true",
                        help="leave the INT8 qkv projection out")
    parser.add_argument("--skip-quantized", action="store_true",
                        help="leave the fused quantize pass and the INT8/FP8 kernel out")
    parser.add_argument("--skip-vsa", action="store_true",
                        help="leave the video sparse attention out")
    parser.add_argument("--vsa-frames", type=int, default=31,
                        help="latent frames of the video sparse attention case (31 is the "
                             "benchmark configuration; fewer for profiler captures)")
    parser.add_argument("--skip-video-layer", action="store_true",
                        help="leave the 125,504-token dense layer on one GPU out")
    parser.add_argument("--no-reference-kernels", action="store_true",
                        help="do not time the reference's own CUDA kernels (oracle/_ref)")
    parser.add_argument("--reference-seconds", type=float, default=60.0,
                        help="about how long the reference arm's warm-up and steps take together")
    parser.add_argument("--dense-only", action="store_true",
                        help="time only the dense BF16 kernel (for profiler captures)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        run_reference(args)
    elif args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_sharded(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
