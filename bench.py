#!/usr/bin/env python
"""Benchmark of the Flux double-stream block forward (bf16, 4096 image + 512 text tokens).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one forward pass of one DoubleStreamBlock (hidden 3072, 24 heads, MLP 12288) over
one image's 4608 tokens.  With N > 1 (launched by torch.distributed.run, one rank per GPU) each
rank runs its own image through a replica of the block: batch data-parallel, no collective on
the data path, weak scaling.  Rank 0 prints one JSON line.

  value     tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e       tokens/s through the public module call with HOST inputs/outputs: pinned-host ->
            device copies of img/txt/vec and a device -> host copy of both outputs every step,
            pipelined over three streams (the module call is a CUDA-graph replay here too)
  roofline  the largest GEMM launch of the step (MLP up-projection of both streams, grouped:
            M=512+4096, K=3072, N=12288, GELU epilogue) timed per launch with CUDA events inside real steps,
            against the measured bf16 peak in MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle (PyTorch fp32 restatement of the reference's block) on the
            host cores, on a bounded sample

`--impl reference` times that CPU path alone (rank 0 only) and prints the same line shape.
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

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "flux_double_block_fwd_tokens_per_s"
UNIT = "tokens/s"
C, H, MLP_RATIO = 3072, 24, 4.0
L_IMG, L_TXT = 4096, 512
GRID = 64
SEED = 2
TOKENS = L_IMG + L_TXT
WORKLOAD = (f"flux_double_stream_block hidden {C}, {H} heads x 128, {L_IMG} image + {L_TXT} text tokens, "
            "batch 1 per GPU, weights N(0,0.02), seed 2")
# Algorithmic work of the timed GEMM launch (2*M*N*K; the MLP up-projections of the text and
# image streams run as one grouped launch, M = 512 + 4096) and of one block step.
DOM_M, DOM_K, DOM_N = TOKENS, C, int(C * MLP_RATIO)
BLOCK_FLOP = 2 * TOKENS * C * (3 * C + C + 2 * int(C * MLP_RATIO)) + 4 * H * TOKENS * TOKENS * (C // H)
NCU_TRAFFIC_BYTES = 193.4e6  # dram read+write bytes per launch of the timed GEMM shape (ncu capture summarised in profiles/)


def make_inputs(seed: int, l_img: int = L_IMG, l_txt: int = L_TXT, grid: int = GRID):
    """Seeded fp32 parameters and activations of the double-stream block config (CPU tensors).

    Parameter names, shapes and draw order are those of the block's own state-dict; weights
    N(0, 0.02), biases 0, QK-norm scales 1, activations and vec N(0, 1).  Nothing here touches
    the oracle: the GPU arm only needs numbers, and the CPU legs feed the same dict to it."""
    from triton_kernels_b200.flux import EmbedND, flux_position_ids
    from triton_kernels_b200.modules import DoubleStreamBlock

    g = torch.Generator().manual_seed(seed)
    with torch.device("meta"):
        shapes = {k: tuple(v.shape) for k, v in DoubleStreamBlock(C, H, MLP_RATIO).state_dict().items()}
    params = {}
    for name, shape in shapes.items():
        if name.endswith(".scale"):
            params[name] = torch.ones(shape)
        elif name.endswith(".bias"):
            params[name] = torch.zeros(shape)
        else:
            params[name] = 0.02 * torch.randn(shape, generator=g)
    img = torch.randn(1, l_img, C, generator=g)
    txt = torch.randn(1, l_txt, C, generator=g)
    vec = torch.randn(1, C, generator=g)
    pe = EmbedND(C // H, 10000, [16, 56, 56])(flux_position_ids(l_txt, l_img // grid, grid))
    return params, img, txt, vec, pe


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU while a region runs.

    Reads NVML directly from a thread every few milliseconds (queries only), so that a timed
    region of some tens of milliseconds still gets samples; falls back to an `nvidia-smi` loop
    when the NVML module is missing."""

    SMI_FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int, period_s: float = 0.004):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples: list[tuple[float, float, int]] = []  # (sm MHz, watts, reason bits)
        self.sm_max = None
        self.proc = None
        self.thread = None
        self._stop = threading.Event()
        self.source = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:  # noqa: BLE001  (older torch without .uuid, or a MIG-style id)
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def start(self):
        try:
            nv, h = self._nvml_handle()
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            bits = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                    "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                    "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
            self._bits = [bits[n] for n in self.REASONS]

            def loop():
                while not self._stop.is_set():
                    try:
                        sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                        watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                        mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                        self.samples.append((sm, watts, sum(1 << i for i, b in enumerate(self._bits) if mask & b)))
                    except Exception:  # noqa: BLE001
                        pass
                    self._stop.wait(self.period_s)

            self.source = "nvml"
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.source = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.SMI_FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read_smi(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm, smax, watts = float(f[1]), float(f[2]), float(f[3])
            except ValueError:
                continue
            self.sm_max = smax
            self.samples.append((sm, watts, sum(1 << i for i, v in enumerate(f[4:8]) if v.lower().startswith("active"))))

    def stop(self) -> dict:
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source (NVML and nvidia-smi unavailable)"]}
        if self.source == "nvml":
            self._stop.set()
            self.thread.join(timeout=2)
        else:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [s[0] for s in self.samples]
        power = [s[1] for s in self.samples]
        mask = 0
        for s in self.samples:
            mask |= s[2]
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_mhz_min": min(sm) if sm else None,
            "sm_max_mhz": self.sm_max,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "source": self.source,
            "reasons": [n for i, n in enumerate(self.REASONS) if mask & (1 << i)],
        }


def bf16_rounded(params, *tensors):
    """The values the GPU arm computes on (parameters and inputs rounded to bf16), as fp32."""
    return {k: v.to(torch.bfloat16).float() for k, v in params.items()}, [t.to(torch.bfloat16).float() for t in tensors]


def cpu_block_time(tokens_img: int, tokens_txt: int, runs: int, warm: int = 1, seed: int = SEED):
    """Median seconds per forward of the CPU oracle's double-stream block (fp32, all host threads)
    on the inputs `make_inputs(seed)` rounded to bf16; also returns the thread count and the
    (img, txt) outputs, which the benchmark compares the GPU step's outputs with."""
    from oracle import flux_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    params, img, txt, vec, pe = make_inputs(seed, tokens_img, tokens_txt, GRID)
    params, (img, txt, vec) = bf16_rounded(params, img, txt, vec)
    times, out = [], None
    with torch.no_grad():
        for i in range(warm + runs):
            t0 = time.perf_counter()
            out = O.double_stream_block(img, txt, vec, pe, params, H)
            if i >= warm:
                times.append(time.perf_counter() - t0)
    return statistics.median(times), torch.get_num_threads(), out


def rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    return float((got - want).norm() / want.norm())


def load_triton_reference():
    """The reference package staged by oracle/make_ref.py, or exits with a one-line reason."""
    from oracle import make_ref

    ref = make_ref.import_reference()
    if ref is None:
        print(json.dumps({"impl": "triton_ref", "unavailable": "oracle/_ref/triton_kernels is not staged "
                          "(run `python oracle/make_ref.py <reference checkout>` where the checkout exists)"}), flush=True)
        raise SystemExit(0)
    return ref


def run_reference(args, rank: int):
    """The reference's own CPU path for the block (its PyTorch blocks, restated in oracle/),
    timed on the host cores; every step is one forward over a bounded token sample."""
    if rank != 0:
        return
    from oracle import flux_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    budget_s = 150.0
    sizes = [(L_IMG, L_TXT), (1024, 128), (256, 64)]
    chosen = sizes[-1]
    per = None
    for li, lt in sizes:
        t, _, _ = cpu_block_time(li, lt, runs=1, warm=0)
        if t * (args.steps + args.warmup) <= budget_s:
            chosen, per = (li, lt), t
            break
    li, lt = chosen
    params, img, txt, vec, pe = make_inputs(SEED, li, lt, GRID)
    with torch.no_grad():
        for _ in range(args.warmup):
            O.double_stream_block(img, txt, vec, pe, params, H)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            O.double_stream_block(img, txt, vec, pe, params, H)
        dt = time.perf_counter() - t0
    value = (li + lt) * args.steps / dt
    sample = f"{args.steps} forward passes of the double-stream block over {li}+{lt} tokens (fp32, torch CPU)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sampled_tokens_per_step": li + lt},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# Per-kernel microbenchmarks at the shapes of the benchmark's kernel config (seed 1):
# (a) RMSNorm [1,4608,3072] and per-head [1,24,4608,128]; (b) LayerNorm+modulation
# [1,4608,3072]; (c) RoPE on q,k [1,24,4608,128]; (d) linear+bias+GELU M=4608 K=3072 N=12288;
# (e) attention [1,24,4608,128]; plus the fused q/k/v assembly and the modulation projection.
# Each kernel is launched back to back over rotating buffer sets that together exceed the
# 126 MB L2, and timed with CUDA events; one JSON line per kernel.
# --------------------------------------------------------------------------------------
def run_micro(which: str, steps: int, warmup: int, impl: str = "b200"):
    """impl "b200": this library's kernels.  impl "triton_ref": the reference's own Triton kernels
    (the staged copy of the reference package) on the same buffers, shapes and timing harness —
    aligned shapes only, the reference's attention kernel has no bounds checks."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    BF = torch.bfloat16
    ours = impl == "b200"
    if ours:
        import triton_kernels_b200  # noqa: F401
        from triton_kernels_b200 import _lib
        from triton_kernels_b200.kernels.attention import attention_into
        from triton_kernels_b200.kernels.linear import linear_into
        from triton_kernels_b200.kernels.normalization import layer_norm_modulation_into
        from triton_kernels_b200.ops.fused import qkv_prepare_into

        lib = _lib.load()
        st = _lib.stream_handle  # evaluated at call time: launches must follow the capturing stream
    else:
        ref = load_triton_reference()
    g = torch.Generator(device=dev).manual_seed(1)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {
        "hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    L, Cc, Hh, D = TOKENS, C, H, C // H

    def randn(*shape, std=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * std).to(BF)

    def time_calls(calls):
        """Seconds per launch.  One pass over all buffer sets is captured in a CUDA graph and
        the graph is replayed, so the host cost of issuing a launch (several microseconds
        through ctypes, comparable to the shortest kernels here) is not part of the number."""
        for c in calls:
            c()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for c in calls:
                    c()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(max(warmup, 1)):
            graph.replay()
        torch.cuda.synchronize()
        reps = max(steps, 1)
        sampler = ClockSampler(0, period_s=0.002)
        sampler.start()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        last_clocks.clear()
        last_clocks.update(sampler.stop())
        return a.elapsed_time(b) * 1e-3 / (reps * len(calls))

    last_clocks: dict = {}  # clock record of the most recent time_calls()

    def sets_for(bytes_per_set):
        return max(2, int(300e6 // bytes_per_set) + 1)

    def emit(name, sec, work, bound):
        if bound == "hbm":
            ach, peak, unit = work / sec / 1e9, peaks["hbm_gbs"], "GB/s"
        else:
            ach, peak, unit = work / sec / 1e12, peaks["bf16_tflops"], "TFLOP/s"
        print(json.dumps({"micro": name, "impl": impl, "us_per_launch": sec * 1e6, "bound": bound, "achieved": ach,
                          "peak": peak, "unit": unit, "frac": ach / peak, "algorithmic_work": work,
                          "sm_mhz": last_clocks.get("sm_mhz"), "sm_mhz_min": last_clocks.get("sm_mhz_min"),
                          "power_w_max": last_clocks.get("power_w_max"), "reasons": last_clocks.get("reasons")}), flush=True)

    def want(name):
        return which in ("all", name)

    if want("layer_norm_modulation"):
        sc, sh = randn(1, Cc, std=0.1), randn(1, Cc, std=0.1)
        bufs = [(randn(L, Cc), torch.empty(L, Cc, device=dev, dtype=BF)) for _ in range(sets_for(2 * L * Cc * 2))]
        if ours:
            calls = [lambda x=x, y=y: layer_norm_modulation_into(x, sc, sh, y, L, 1e-6) for x, y in bufs]
        else:
            calls = [lambda x=x: ref.layer_norm_modulation(x.view(1, L, Cc), sc.view(1, 1, Cc), sh.view(1, 1, Cc), 1e-6)
                     for x, _ in bufs]
        emit("layer_norm_modulation[1,4608,3072]", time_calls(calls), 2 * L * Cc * 2 + 2 * Cc * 2, "hbm")
        if ours:
            # The same kernel on a problem 16x larger, and a plain device copy of both sizes: a 57 MB
            # problem is over in ~10 us and cannot reach the bandwidth of a multi-GB stream.
            Lb = 16 * L
            xb, yb = randn(Lb, Cc), torch.empty(Lb, Cc, device=dev, dtype=BF)
            emit("layer_norm_modulation[1,73728,3072]", time_calls([lambda: layer_norm_modulation_into(xb, sc, sh, yb, Lb, 1e-6)]),
                 2 * Lb * Cc * 2, "hbm")
            emit("device_copy[73728,3072] (torch, for scale)", time_calls([lambda: yb.copy_(xb)]), 2 * Lb * Cc * 2, "hbm")
            calls = [lambda x=x, y=y: y.copy_(x) for x, y in bufs]
            emit("device_copy[4608,3072] (torch, for scale)", time_calls(calls), 2 * L * Cc * 2, "hbm")
            del xb, yb
    if want("rms_norm"):
        w = torch.ones(Cc, device=dev, dtype=BF)
        wh = torch.ones(D, device=dev, dtype=BF)
        bufs = [(randn(L, Cc), torch.empty(L, Cc, device=dev, dtype=BF)) for _ in range(sets_for(2 * L * Cc * 2))]
        if ours:
            calls = [lambda x=x, y=y: lib.fluxb_rms_norm(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, 1, 1, L, Cc, 0, 0, Cc,
                                                          1e-6, 1, st()) for x, y in bufs]
            calls_h = [lambda x=x, y=y: lib.fluxb_rms_norm(x.data_ptr(), wh.data_ptr(), y.data_ptr(), None, 1, 1, L * Hh, D, 0,
                                                            0, D, 1e-6, 1, st()) for x, y in bufs]
        else:
            calls = [lambda x=x: ref.rms_norm(x.view(1, L, Cc), w) for x, _ in bufs]
            calls_h = [lambda x=x: ref.rms_norm(x.view(1, Hh, L, D), wh) for x, _ in bufs]
        emit("rms_norm[1,4608,3072]", time_calls(calls), 2 * L * Cc * 2, "hbm")
        emit("rms_norm[1,24,4608,128]", time_calls(calls_h), 2 * L * Cc * 2, "hbm")
    pe = torch.randn(L, D // 2, 2, 2, device=dev, generator=g)
    if want("rope"):
        bufs = [tuple(randn(Hh, L, D) for _ in range(2)) + tuple(torch.empty(Hh, L, D, device=dev, dtype=BF) for _ in range(2))
                for _ in range(sets_for(4 * L * Cc * 2))]
        if ours:
            calls = [lambda q=q, k=k, oq=oq, ok=ok: lib.fluxb_rope(q.data_ptr(), k.data_ptr(), pe.data_ptr(), oq.data_ptr(),
                                                                     ok.data_ptr(), Hh, L, D, 1, st()) for q, k, oq, ok in bufs]
        else:
            pe6 = pe.view(1, 1, L, D // 2, 2, 2)
            calls = [lambda q=q, k=k: ref.apply_rope(q.view(1, Hh, L, D), k.view(1, Hh, L, D), pe6) for q, k, _, _ in bufs]
        emit("rope[1,24,4608,128]", time_calls(calls), 4 * L * Cc * 2 + pe.numel() * 4, "hbm")
    if want("qkv_prepare") and ours:
        wh = torch.ones(D, device=dev, dtype=BF)
        bufs = [(randn(1, L, 3 * Cc),) + tuple(torch.empty(1, Hh, L, D, device=dev, dtype=BF) for _ in range(3))
                for _ in range(sets_for(6 * L * Cc * 2))]
        calls = [lambda s_=s_, q=q, k=k, v=v: qkv_prepare_into([(s_, wh, wh)], pe, q, k, v, Hh) for s_, q, k, v in bufs]
        emit("qkv_prepare[1,4608,9216]", time_calls(calls), 6 * L * Cc * 2 + pe.numel() * 4, "hbm")
    if want("modulation_projection"):
        vec = randn(1, Cc)
        bufs = [(randn(6 * Cc, Cc, std=0.02), randn(6 * Cc, std=0.02), torch.empty(1, 6 * Cc, device=dev, dtype=BF))
                for _ in range(3)]
        if ours:
            calls = [lambda w=w, b=b, o=o: lib.fluxb_modulation_gemv(vec.data_ptr(), w.data_ptr(), b.data_ptr(), o.data_ptr(), 1,
                                                                      6 * Cc, Cc, 1, st()) for w, b, o in bufs]
        else:  # the reference's Modulation: silu, then its linear kernel with M = batch
            calls = [lambda w=w, b=b: ref.linear(torch.nn.functional.silu(vec), w, b) for w, b, _ in bufs]
        emit("modulation_projection[18432x3072]", time_calls(calls), 6 * Cc * Cc * 2, "hbm")
    if want("linear_gelu"):
        M, K, N = L, Cc, 4 * Cc
        bufs = [(randn(M, K), randn(N, K, std=0.02), randn(N, std=0.02), torch.empty(M, N, device=dev, dtype=BF))
                for _ in range(2)]
        if ours:
            calls = [lambda x=x, w=w, b=b, y=y: linear_into(x, w, b, y, epi=_lib.EPI_GELU) for x, w, b, y in bufs]
        else:
            calls = [lambda x=x, w=w, b=b: ref.linear(x, w, b, activation="GELU") for x, w, b, _ in bufs]
        emit("linear_bias_gelu[M4608,K3072,N12288]", time_calls(calls), 2.0 * M * N * K, "tensor")
    if want("linear_down") and ours:
        # the other GEMMs of a block step as it launches them: both streams grouped, gate/residual epilogue
        from triton_kernels_b200.kernels.linear import linear_grouped_into
        Lt_, Li_ = 512, L - 512
        for name, K_ in (("linear_proj_gate_resid[M512+4096,K3072,N3072]", Cc), ("linear_mlp_down_gate_resid[M512+4096,K12288,N3072]", 4 * Cc)):
            bufs = []
            for _ in range(2):
                probs = []
                for M_ in (Lt_, Li_):
                    probs.append(dict(x2d=randn(M_, K_), w=randn(Cc, K_, std=0.02), b=randn(Cc, std=0.02),
                                      y=torch.empty(M_, Cc, device=dev, dtype=BF), resid=randn(M_, Cc), gate=randn(1, Cc),
                                      gate_stride=0, rows_per_batch=M_))
                bufs.append(probs)
            calls = [lambda pr=pr: linear_grouped_into(pr, epi=_lib.EPI_GATE_RESID) for pr in bufs]
            emit(name, time_calls(calls), 2.0 * L * Cc * K_, "tensor")
    if want("linear_qkv") and ours:
        # both streams' q|k|v projection with QK norm, RoPE and the head-major layout in the epilogue
        from triton_kernels_b200.kernels.linear import linear_qkv_grouped_into
        Lt_, Li_ = 512, L - 512
        ones = torch.ones(D, device=dev, dtype=BF)
        pe6 = pe.view(1, 1, L, D // 2, 2, 2)
        bufs = [([randn(1, Lt_, Cc), randn(1, Li_, Cc)], [randn(3 * Cc, Cc, std=0.02) for _ in range(2)],
                 torch.empty(3, 1, Hh, L, D, device=dev, dtype=BF)) for _ in range(2)]
        calls = [lambda xs=xs, ws=ws, o=o: linear_qkv_grouped_into(
            [dict(x=x, w=w, b=None, q_scale=ones, k_scale=ones) for x, w in zip(xs, ws)], pe6, o) for xs, ws, o in bufs]
        emit("linear_qkv_heads[M512+4096,K3072,N9216]", time_calls(calls), 2.0 * L * 3 * Cc * Cc, "tensor")
    if want("attention"):
        bufs = [tuple(randn(1, Hh, L, D) for _ in range(3)) + (torch.empty(1, L, Hh, D, device=dev, dtype=BF),)
                for _ in range(3)]
        if ours:
            calls = [lambda q=q, k=k, v=v, o=o: attention_into(q, k, v, o.permute(0, 2, 1, 3), D ** -0.5) for q, k, v, o in bufs]
        else:
            calls = [lambda q=q, k=k, v=v: ref.scaled_dot_product_attention(q, k, v) for q, k, v, _ in bufs]
        emit("attention[1,24,4608,128]", time_calls(calls), 4.0 * Hh * L * L * D, "tensor")
    if ours:
        code, where = _lib.device_status()
        if code != 0:
            raise SystemExit(f"device status word reports error {code} at {where}")


# --------------------------------------------------------------------------------------
# Full Flux DiT denoising step (19 double + 38 single blocks, 4096 + 512 tokens, batch 1,
# weights N(0,0.02) drawn on the device with seed 3).  `dit_measure` returns the step latency
# with device-resident inputs (eager and CUDA-graph replay) and end to end with host buffers:
# every step copies the latent tokens [1,4096,64], the text tokens [1,512,4096], timestep and
# guidance from pinned host memory to the device and the prediction [1,4096,64] back.
# --------------------------------------------------------------------------------------
DIT_FLOP = (19 + 38) * BLOCK_FLOP + 2 * L_IMG * 64 * C * 2 + 2 * L_TXT * 4096 * C


def _init_flux_weights(model, dev, g):
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if name.endswith(".scale"):
                prm.fill_(1.0)
            elif name.endswith(".bias"):
                prm.zero_()
            else:
                prm.copy_((torch.randn(prm.shape, device=dev, generator=g) * 0.02).to(prm.dtype))


def _reference_dit(ref, depth: int, depth_single: int):
    """The benchmark's DiT assembled from the reference's own parts: its Triton-kernel blocks
    (triton_kernels/modules/blocks.py:78-172) between its PyTorch embedders and last layer
    (triton_kernels/flux/layers.py:55-85, 267-278).  The reference has no model class."""
    from torch import nn

    import importlib

    RL = importlib.import_module(ref.__name__ + ".flux.layers")  # the staged copy's PyTorch layers

    class RefDiT(nn.Module):
        def __init__(self):
            super().__init__()
            self.img_in = nn.Linear(64, C)
            self.time_in = RL.MLPEmbedder(256, C)
            self.guidance_in = RL.MLPEmbedder(256, C)
            self.txt_in = nn.Linear(4096, C)
            self.double_blocks = nn.ModuleList([ref.DoubleStreamBlock(C, H, MLP_RATIO) for _ in range(depth)])
            self.single_blocks = nn.ModuleList([ref.SingleStreamBlock(C, H, MLP_RATIO) for _ in range(depth_single)])
            self.final_layer = RL.LastLayer(C, 1, 64)

        def forward(self, img, txt, t, gd, pe):
            # the reference's timestep_embedding builds its frequencies on the host on every call
            # (triton_kernels/flux/layers.py:66), which a CUDA-graph capture cannot contain; this
            # package's device-side form of the same formula stands in for it
            from triton_kernels_b200.flux.model import timestep_embedding

            img = self.img_in(img)
            vec = self.time_in(timestep_embedding(t, 256).to(img.dtype))
            vec = vec + self.guidance_in(timestep_embedding(gd, 256).to(img.dtype))
            txt = self.txt_in(txt)
            for blk in self.double_blocks:
                img, txt = blk(img=img, txt=txt, vec=vec, pe=pe)
            x = torch.cat((txt, img), 1)
            for blk in self.single_blocks:
                x = blk(x, vec=vec, pe=pe)
            return self.final_layer(x[:, txt.shape[1]:], vec)

    return RefDiT()


def dit_measure(dev, steps: int, warmup: int, depth: int = 19, depth_single: int = 38, impl: str = "b200",
                barrier=None, max_over_ranks=None) -> dict:
    from triton_kernels_b200.flux import EmbedND, GraphedForward, flux_position_ids

    BF = torch.bfloat16
    barrier = barrier or torch.cuda.synchronize
    max_over_ranks = max_over_ranks or (lambda x: x)
    g = torch.Generator(device=dev).manual_seed(3)
    if impl == "b200":
        from triton_kernels_b200 import _lib
        from triton_kernels_b200.flux import FluxDiT, FluxParams

        with torch.device(dev):
            model = FluxDiT(FluxParams(depth=depth, depth_single_blocks=depth_single)).to(BF)
    else:
        ref = load_triton_reference()
        with torch.device(dev):
            model = _reference_dit(ref, depth, depth_single).to(BF)
    _init_flux_weights(model, dev, g)
    img = torch.randn(1, L_IMG, 64, device=dev, generator=g).to(BF)
    txt = torch.randn(1, L_TXT, 4096, device=dev, generator=g).to(BF)
    t = torch.tensor([0.5], device=dev)
    gd = torch.tensor([3.5], device=dev)
    pe = EmbedND(128, 10000, [16, 56, 56])(flux_position_ids(L_TXT, GRID, GRID, device=dev))
    fwd = lambda i, x, tt, gg: model(i, x, tt, gg, pe)

    def timed(fn, n=steps):
        for _ in range(max(warmup, 1)):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(max(n, 1)):
            out = fn()
        b.record()
        barrier()
        return max_over_ranks(a.elapsed_time(b)) / max(n, 1), out

    with torch.no_grad():
        launches = None
        if impl == "b200":
            calls0 = _lib.kernel_calls
            fwd(img, txt, t, gd)
            launches = _lib.kernel_calls - calls0
        else:
            fwd(img, txt, t, gd)  # compiles and autotunes the Triton kernels
        eager_ms, out = timed(lambda: fwd(img, txt, t, gd), n=min(steps, 5))
        graphed = GraphedForward(fwd, (img, txt, t, gd))
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        graph_ms, out_g = timed(lambda: graphed(img, txt, t, gd))
        clocks = sampler.stop()
        same = bool(torch.equal(out, out_g))

        # end to end: pinned host inputs in, prediction out, every step, on the compute stream
        # (5 MB per step against tens of milliseconds of kernels: nothing to overlap)
        host_in = [x.cpu().pin_memory() for x in (img, txt, t, gd)]
        host_out = torch.empty_like(out_g, device="cpu").pin_memory()
        stat = graphed.static_inputs

        def e2e_step():
            for dst, src in zip(stat, host_in):
                dst.copy_(src, non_blocking=True)
            graphed.graph.replay()
            host_out.copy_(graphed.static_outputs, non_blocking=True)
            return host_out

        e2e_ms, _ = timed(e2e_step)
        torch.cuda.synchronize()
        e2e_same = bool(torch.equal(host_out, out_g.cpu()))
    rec = {
        "workload": f"flux_dit_step {depth} double + {depth_single} single blocks, {L_IMG}+{L_TXT} tokens, batch 1 per GPU, "
                    "bf16, weights N(0,0.02), seed 3",
        "impl": impl,
        "ms_per_step": graph_ms, "ms_per_step_eager": eager_ms, "launch": "cuda graph replay",
        "tokens_per_s_per_gpu": TOKENS / (graph_ms * 1e-3),
        "tflop_per_step": DIT_FLOP / 1e12, "tflops_achieved": DIT_FLOP / (graph_ms * 1e-3) / 1e12,
        "e2e": {"ms_per_step": e2e_ms, "tokens_per_s_per_gpu": TOKENS / (e2e_ms * 1e-3),
                "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in host_in),
                "d2h_bytes_per_step": host_out.numel() * host_out.element_size(),
                "output_equals_device_resident_run": e2e_same},
        "output_finite": bool(torch.isfinite(out_g.float()).all()), "graph_equals_eager": same,
        "params_gb": sum(p.numel() for p in model.parameters()) * 2 / 1e9,
        "clocks": clocks,
    }
    if launches is not None:
        rec["kernel_calls_per_step"] = launches
        code, where = _lib.device_status()
        rec["device_status"] = [code, where]
    del graphed, model
    torch.cuda.empty_cache()
    return rec


def run_dit(steps: int, warmup: int, impl: str = "b200"):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    print(json.dumps(dit_measure(dev, steps, warmup, impl=impl)), flush=True)


# --------------------------------------------------------------------------------------
# Ulysses sequence parallelism (benchmark config 5b): ONE double-stream block over a
# 128x128-patch image (16384 image + 512 text tokens, batch 1) with the tokens sharded over the
# ranks and an all-to-all on heads around attention.  Strong scaling: the total work is fixed.
# --------------------------------------------------------------------------------------
def ulysses_measure(rank: int, local_rank: int, world: int, steps: int, warmup: int, exchange: str,
                    single_rank_baseline: bool = False, scatter_from_projection: bool = False,
                    no_graph: bool = False) -> dict:
    """One double-stream block over 16384 image + 512 text tokens with the tokens sharded over the
    ranks of the default process group (which the caller has initialised when world > 1).  With
    `single_rank_baseline` every rank first times the unsharded block on its own GPU, so that the
    record carries the strong-scaling efficiency t_1 / (P * t_P) measured in the same process."""
    import torch.distributed as dist

    import triton_kernels_b200 as tk
    from triton_kernels_b200 import _lib
    from triton_kernels_b200.flux import EmbedND, flux_position_ids
    from triton_kernels_b200.parallel import SequenceParallel, shard_joint_sequence

    dev = torch.device("cuda", local_rank)
    BF = torch.bfloat16
    li, lt, grid = 16384, 512, 128
    warmup = max(warmup, 3)
    g = torch.Generator(device=dev).manual_seed(4)  # same parameters and inputs on every rank
    with torch.device(dev):
        block = tk.DoubleStreamBlock(C, H, MLP_RATIO).to(BF)
    _init_flux_weights(block, dev, g)
    img = torch.randn(1, li, C, device=dev, generator=g).to(BF)
    txt = torch.randn(1, lt, C, device=dev, generator=g).to(BF)
    vec = torch.randn(1, C, device=dev, generator=g).to(BF)
    pe = EmbedND(128, 10000, [16, 56, 56])(flux_position_ids(lt, grid, grid, device=dev))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn):
        """Milliseconds per step, max over ranks.  The one-GPU step is four to eight times longer
        than a sharded one, so equal step counts would time the former at the power cap and the
        latter in the first, faster milliseconds after it: every form is therefore warmed up for
        at least 0.25 s and timed over at least 0.25 s (never fewer than `warmup` / `steps` steps;
        the counts come from an all-reduced estimate, so all ranks run the same number)."""
        for _ in range(3):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            fn()
        e1.record()
        barrier()
        est_ms = max(max_over_ranks(e0.elapsed_time(e1)) / 3, 1e-3)
        n_warm = max(warmup, int(250.0 / est_ms) + 1)
        n_timed = max(steps, int(250.0 / est_ms) + 1)
        for _ in range(n_warm):
            fn()
        barrier()
        e0.record()
        for _ in range(n_timed):
            fn()
        e1.record()
        barrier()
        counts["steps"] = n_timed
        counts["warmup"] = n_warm + 6
        return max_over_ranks(e0.elapsed_time(e1)) / n_timed

    counts: dict = {}

    single_ms = None
    with torch.no_grad():
        if single_rank_baseline or world == 1:
            single_ms = timed(lambda: block(img, txt, vec, pe))
        if world > 1:
            sp = block.sequence_parallel = SequenceParallel(exchange=exchange, scatter_from_projection=scatter_from_projection)
            txt_l, img_l, pe_l = shard_joint_sequence(txt, img, pe, rank, world)
            del img, txt
            calls0 = _lib.kernel_calls
            block(img_l, txt_l, vec, pe_l)
            launches = _lib.kernel_calls - calls0
            step = lambda: block(img_l, txt_l, vec, pe_l)
            launch = "eager"
            if exchange == "peer" and not no_graph:
                # The peer exchange is kernels only (its barriers keep their epochs in the arena), so
                # the sharded step replays from a CUDA graph like the single-GPU step does; every
                # rank replays the same number of times.
                from triton_kernels_b200.flux import GraphedForward

                graphed = GraphedForward(lambda i, t, v: block(i, t, v, pe_l), (img_l, txt_l, vec))
                step = graphed.graph.replay  # the captured inputs already hold this rank's shard
                launch = "cuda graph replay"
            sampler = ClockSampler(local_rank)
            sampler.start()
            ms = timed(step)
            clocks = sampler.stop()
            sp.check()
        else:
            ms, launches, clocks, launch = single_ms, None, None, "eager"
    tokens = li + lt
    flop = 2 * tokens * C * (3 * C + C + 2 * int(C * MLP_RATIO)) + 4 * H * tokens * tokens * (C // H)
    rec = {
        "workload": f"flux_double_stream_block hidden {C}, {H} heads x 128, {li} image + {lt} text tokens, batch 1 in total, "
                    "weights N(0,0.02), seed 4",
        "parallelism": f"ulysses sequence-parallel x{world}", "scaling": "strong",
        "exchange": (("stores into peer memory from the producing kernels"
                      + (" (q|k|v from the projection's epilogue)" if scatter_from_projection else ""))
                     if exchange == "peer" else "NCCL all-to-all") if world > 1 else None,
        "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3), "steps": counts.get("steps", steps),
        "warmup": counts.get("warmup", warmup), "launch": launch,
        "timing": "each form warmed up for at least 0.25 s and timed over at least 0.25 s, so that the one-GPU step and the "
                  "shorter sharded steps are all measured in the same (power-capped) regime",
        "block_tflop": flop / 1e12, "tflops_per_gpu": flop / (ms * 1e-3) / 1e12 / world,
    }
    if single_ms is not None:
        rec["single_gpu_ms_per_step"] = single_ms
        rec["efficiency_vs_single_gpu"] = single_ms / (world * ms)
    if world > 1:
        # Bytes each GPU sends over NVLink per block: (P-1)/P of its q, k, v and of its attention output.
        l_loc = tokens // world
        rec["nvlink_bytes_sent_per_gpu_per_step"] = (world - 1) / world * (3 + 1) * l_loc * C * 2
        rec["kernel_calls_per_step"] = launches
        rec["clocks"] = clocks
        if exchange == "peer":
            # The assembly kernel alone (it IS the q/k/v transfer): event-timed, barriers kept in step.
            from triton_kernels_b200.ops.fused import qkv_prepare_scatter
            pb = sp.peer_buffers(1, l_loc, H, C // H, BF)
            qkv_t = torch.randn(1, lt // world, 3 * C, device=dev, generator=g).to(BF)
            qkv_i = torch.randn(1, li // world, 3 * C, device=dev, generator=g).to(BF)
            streams = [(qkv_t, block.txt_attn.norm.query_norm.scale, block.txt_attn.norm.key_norm.scale),
                       (qkv_i, block.img_attn.norm.query_norm.scale, block.img_attn.norm.key_norm.scale)]
            times = []
            for _ in range(8):
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                dist.barrier()
                a0.record()
                qkv_prepare_scatter(streams, pe_l, pb.q_bases, pb.P, pb.k_off, pb.v_off, H, C // H, pb.qkv_strides)
                a1.record()
                for b in (0, 1):
                    pb.arena.signal(b)
                    pb.arena.wait(b)
                torch.cuda.synchronize()
                times.append(a0.elapsed_time(a1))
            t_asm = max_over_ranks(sorted(times)[len(times) // 2])
            qkv_sent = (world - 1) / world * 3 * l_loc * C * 2
            rec["assembly_scatter_kernel_ms"] = t_asm
            rec["assembly_scatter_nvlink_gbs_per_gpu"] = qkv_sent / (t_asm * 1e-3) / 1e9
        sp.check()
        sp.close()
        block.sequence_parallel = None
    code, where = _lib.device_status()
    if code != 0:
        raise SystemExit(f"device status word reports error {code} at {where}")
    del block
    torch.cuda.empty_cache()
    return rec


def run_ulysses(args, rank: int, local_rank: int, world: int):
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    rec = ulysses_measure(rank, local_rank, world, args.steps, args.warmup, args.exchange, single_rank_baseline=True,
                          scatter_from_projection=args.sp_scatter_from_projection, no_graph=args.no_graph)
    if rank == 0:
        print(json.dumps({
            "metric": "flux_double_block_fwd_tokens_per_s", "value": rec["tokens_per_s"], "unit": UNIT,
            "n_gpus": world, "steps": rec["steps"], "warmup": rec["warmup"], "ms_per_step": rec["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": rec, "gpu_launches": (rec.get("kernel_calls_per_step") or 0) * rec["steps"],
            "clocks": rec.get("clocks"),
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# Sequence-length sweeps with the shapes of the reference's own benchmark scripts
# (benchmarks/{linear,attention,layer_norm,rms_norm,rope}.py: batch 4, 24 heads x 128,
# hidden 3072; seq_len 256..4096 step 256, linear 64..2048 step 64; fp32 inputs for the norm
# and RoPE kernels, bf16 for linear and attention), through the public operator API.  Each
# line carries the reference's figure of merit, "GB/s" = 2 * numel(x) * element_size / time
# (for every kernel, also the GEMM and attention), and the real work rate of the kernel.
# Timing like triton.testing.do_bench: L2 flushed before every call, median of the calls.
# --------------------------------------------------------------------------------------
def run_sweep(which: str, reps: int):
    import triton_kernels_b200 as tk
    from triton_kernels_b200 import _lib

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    B, Hh, D, E = 4, H, C // H, C

    def randn(*shape, dtype=torch.float32):
        return torch.randn(*shape, device=dev, generator=g).to(dtype)

    def median_ms(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(max(reps, 5)):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    def emit(kernel, seq, ms, x, work, unit):
        print(json.dumps({"sweep": kernel, "batch": B, "seq_len": seq, "ms": ms,
                          "reference_gbps": 2 * x.numel() * x.element_size() / ms * 1e-6,
                          "work_rate": work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9), "unit": unit}), flush=True)

    seqs = [256 * i for i in range(1, 17)]
    if which in ("all", "linear"):
        w, b = randn(E, E, dtype=torch.bfloat16), randn(E, dtype=torch.bfloat16)
        for seq in [64 * i for i in range(1, 33)]:
            x = randn(B, seq, E, dtype=torch.bfloat16)
            emit("linear", seq, median_ms(lambda: tk.linear(x, w, b)), x, 2.0 * B * seq * E * E, "TFLOP/s")
    if which in ("all", "attention"):
        for seq in seqs:
            q, k, v = (randn(B, Hh, seq, D, dtype=torch.bfloat16) for _ in range(3))
            emit("attention", seq, median_ms(lambda: tk.scaled_dot_product_attention(q, k, v)), q,
                 4.0 * B * Hh * seq * seq * D, "TFLOP/s")
    if which in ("all", "layer_norm"):
        for seq in seqs:
            x, sc, sh = randn(B, seq, E), randn(B, 1, E), randn(B, 1, E)
            emit("layer_norm_modulation", seq, median_ms(lambda: tk.layer_norm_modulation(x, sc, sh)), x,
                 2.0 * x.numel() * 4, "GB/s")
    if which in ("all", "rms_norm"):
        for seq in seqs:
            x, sc = randn(B, Hh, seq, D), randn(D)
            emit("rms_norm", seq, median_ms(lambda: tk.rms_norm(x, sc)), x, 2.0 * x.numel() * 4, "GB/s")
    if which in ("all", "rope"):
        for seq in seqs:
            q, k, pe = randn(B, Hh, seq, D), randn(B, Hh, seq, D), randn(1, 1, seq, D // 2, 2, 2)
            emit("rope", seq, median_ms(lambda: tk.apply_rope(q, k, pe)), q, 4.0 * q.numel() * 4 + pe.numel() * 4, "GB/s")
    code, where = _lib.device_status()
    if code != 0:
        raise SystemExit(f"device status word reports error {code} at {where}")


def traffic_from_profile():
    """DRAM bytes per launch of the timed GEMM shape, from the ncu summary committed for it (a line
    `traffic_bytes_per_launch: <number>` written when the capture was summarised)."""
    import re

    path = ROOT / "profiles" / "gemm_pair_kernel_linear_gelu_M4608_K3072_N12288.md"
    try:
        m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)", path.read_text())
        return (float(m.group(1)), f"profiles/{path.name}") if m else (None, None)
    except OSError:
        return None, None


def host_copy_probe(dev, barrier, max_over_ranks, nbytes: int = 28311552, reps: int = 10) -> dict:
    """Pinned host <-> device copy rate of this process with every rank copying at the same time
    (one cudaMemcpyAsync per buffer, the way the end-to-end leg moves a step's image tokens)."""
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = {"bytes": nbytes}
    for name, (dst, src) in (("h2d", (d, h)), ("d2h", (h, d))):
        dst.copy_(src, non_blocking=True)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        b.record()
        barrier()
        out[f"{name}_gbs_per_gpu"] = nbytes * reps / (max_over_ranks(a.elapsed_time(b)) * 1e-3) / 1e9
    # both directions at once, on two streams
    s2 = torch.cuda.Stream(dev)
    h2 = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d2 = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    s2.wait_stream(torch.cuda.current_stream())
    for _ in range(reps):
        d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            h2.copy_(d2, non_blocking=True)
    torch.cuda.current_stream().wait_stream(s2)
    b.record()
    barrier()
    out["both_directions_gbs_per_gpu_each_way"] = nbytes * reps / (max_over_ranks(a.elapsed_time(b)) * 1e-3) / 1e9
    return out


def run_triton_ref_block(args):
    """The reference's own DoubleStreamBlock (its Triton kernels, stock code path) on the
    benchmark's workload, one GPU: the bar this library is meant to beat.  Same seeded weights and
    inputs; timed eagerly as the reference's scripts do (scripts/double_triton.py:43-67) and as a
    CUDA-graph replay, which removes its host-side launch work."""
    from triton_kernels_b200.flux import GraphedForward

    ref = load_triton_reference()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    BF = torch.bfloat16
    params, img, txt, vec, pe = make_inputs(SEED)
    block = ref.DoubleStreamBlock(C, H, MLP_RATIO).to(BF)
    block.load_state_dict({k: v.to(BF) for k, v in params.items()})
    block = block.to(dev)
    img_d, txt_d, vec_d, pe_d = img.to(BF).to(dev), txt.to(BF).to(dev), vec.to(BF).to(dev), pe.to(dev)
    call = lambda i, t, v: block(img=i, txt=t, vec=v, pe=pe_d)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            out = fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps, out

    with torch.no_grad():
        call(img_d, txt_d, vec_d)  # compiles and autotunes
        eager_ms, out = timed(lambda: call(img_d, txt_d, vec_d))
        graph_ms = None
        try:
            graphed = GraphedForward(call, (img_d, txt_d, vec_d))
            sampler = ClockSampler(0)
            sampler.start()
            graph_ms, out = timed(lambda: graphed(img_d, txt_d, vec_d))
            clocks = sampler.stop()
        except Exception as e:  # noqa: BLE001  (a launcher that cannot be captured: keep the eager number)
            clocks = {"note": f"graph capture failed: {e!r}"}
    ms = min(eager_ms, graph_ms) if graph_ms is not None else eager_ms
    line = {
        "impl": "triton_ref", "metric": METRIC, "value": TOKENS / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "ms_per_step_eager": eager_ms,
        "ms_per_step_graph": graph_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "block_tflops_achieved": BLOCK_FLOP / (ms * 1e-3) / 1e12,
                   "implementation": "reference DoubleStreamBlock on its own Triton kernels (staged copy of the reference package)"},
        "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        _, _, want = cpu_block_time(L_IMG, L_TXT, runs=1, warm=0)
        line["parity"] = {"rel_l2_img": rel_l2(out[0], want[0]), "rel_l2_txt": rel_l2(out[1], want[1]),
                          "against": "fp32 CPU oracle on the same bf16-rounded weights and inputs"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "triton_ref"],
                    help="b200: this library (default).  reference: the reference's CPU path (its PyTorch blocks) on the "
                         "host cores.  triton_ref: the reference's own Triton kernels on one GPU (block, --micro, --dit)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle legs (baseline timing and parity)")
    ap.add_argument("--no-graph", action="store_true", help="time eager module calls instead of CUDA-graph replays")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sub-records (sustained replay, full DiT step, Ulysses block, host copy probe)")
    ap.add_argument("--parallel", default="dp", choices=["dp", "ulysses"],
                    help="multi-GPU sharding: batch data-parallel (default, weak scaling) or Ulysses sequence parallelism "
                         "on a 16384+512-token block (strong scaling)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="--parallel ulysses: how heads and tokens are exchanged around attention: stores into peer "
                         "memory from the producing kernels (default) or two NCCL all-to-alls")
    ap.add_argument("--sp-scatter-from-projection", action="store_true",
                    help="--parallel ulysses with the peer exchange: the q|k|v projection's epilogue stores into the peers' "
                         "arenas itself instead of the assembly kernel after it (measured slower on two GPUs)")
    ap.add_argument("--sweep", default=None, help="sequence-length sweep with the reference benchmark scripts' shapes: "
                    "all | linear | attention | layer_norm | rms_norm | rope (--steps = timed calls per point)")
    ap.add_argument("--dit", action="store_true", help="time the full 19+38 block DiT step instead of one block")
    ap.add_argument("--micro", default=None, help="per-kernel microbenchmark: all | linear_qkv | layer_norm_modulation | rms_norm | "
                    "rope | qkv_prepare | modulation_projection | linear_gelu | linear_down | attention")
    args = ap.parse_args()
    gpu_impl = "triton_ref" if args.impl == "triton_ref" else "b200"
    if args.micro:
        with torch.no_grad():
            run_micro(args.micro, args.steps, args.warmup, gpu_impl)
        return
    if args.dit:
        run_dit(args.steps, args.warmup, gpu_impl)
        return
    if args.sweep:
        run_sweep(args.sweep, args.steps)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.impl == "triton_ref":
        if rank == 0:
            run_triton_ref_block(args)
        return
    if args.parallel == "ulysses":
        run_ulysses(args, rank, local_rank, world)
        return

    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime

        # a short collective timeout: a rank that fails inside a sub-record ends the others' next
        # collective with an error (recorded in the line) instead of stalling the run
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    import triton_kernels_b200 as tk
    from triton_kernels_b200 import _lib
    import triton_kernels_b200.modules.blocks as blocks_mod

    _lib.load()
    BF = torch.bfloat16
    params, img, txt, vec, pe = make_inputs(SEED + rank)  # each rank has its own image
    block = tk.DoubleStreamBlock(C, H, MLP_RATIO).to(BF)
    block.load_state_dict({k: v.to(BF) for k, v in params.items()})
    block = block.to(dev)
    img_h, txt_h, vec_h = (t.to(BF).pin_memory() for t in (img, txt, vec))
    img_d, txt_d, vec_d, pe_d = img_h.to(dev), txt_h.to(dev), vec_h.to(dev), pe.to(dev)
    del params, img, txt, vec

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- device-resident timing
    # The step is the public module call; by default it is captured once in a CUDA graph and
    # replayed (11 kernel launches per replay), which removes the host-side launch work.
    from triton_kernels_b200.flux import GraphedForward

    with torch.no_grad():
        for _ in range(args.warmup):
            block(img_d, txt_d, vec_d, pe_d)
        calls0 = _lib.kernel_calls
        block(img_d, txt_d, vec_d, pe_d)
        launches_per_step = _lib.kernel_calls - calls0
        graphed = None
        if args.no_graph:
            step = lambda: block(img_d, txt_d, vec_d, pe_d)
        else:
            graphed = GraphedForward(lambda i, t, v: block(i, t, v, pe_d), (img_d, txt_d, vec_d))
            step = lambda: graphed(img_d, txt_d, vec_d)
        for _ in range(args.warmup):
            step()
        sampler = ClockSampler(local_rank)
        sampler.start()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out_step = step()
        e1.record()
        barrier()
        launches = launches_per_step * args.steps
        ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop()
        out_img_h, out_txt_h = out_step[0].float().cpu(), out_step[1].float().cpu()  # checked against the oracle below

        # ------------------------------------------------------------ dominant kernel, per launch
        # The grouped MLP up-projection of both streams is wrapped with CUDA events for a few eager
        # steps that directly follow the timed region, with the SM clock sampled while they run.
        probe = []
        grouped_launch = blocks_mod.linear_grouped_into

        def probed_launch(problems, **kw):
            n, k = problems[0]["w"].shape
            if (sum(p["x2d"].shape[0] for p in problems), n, k) == (DOM_M, DOM_N, DOM_K) and kw.get("epi") == _lib.EPI_GELU:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                grouped_launch(problems, **kw)
                b.record()
                probe.append((a, b))
            else:
                grouped_launch(problems, **kw)

        blocks_mod.linear_grouped_into = probed_launch
        dom_sampler = ClockSampler(local_rank)
        dom_sampler.start()
        try:
            for _ in range(max(args.steps, 20)):
                block(img_d, txt_d, vec_d, pe_d)
            torch.cuda.synchronize()
        finally:
            blocks_mod.linear_grouped_into = grouped_launch
        dom_clocks = dom_sampler.stop()
        durs = [a.elapsed_time(b) for a, b in probe]
        dom_ms = sum(durs) / len(durs)

        # ------------------------------------------------------------ end to end with host buffers
        # Two captured copies of the module call, each with its own device-side input and output
        # buffers, so that step i+1's host->device copy and step i-1's device->host copy run
        # under step i's kernels.  (--no-graph: eager module calls on fresh tensors instead.)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        s_cmp = torch.cuda.current_stream()
        bufs = [[torch.empty_like(img_d), torch.empty_like(txt_d), torch.empty_like(vec_d)] for _ in range(2)]
        outs_h = [[torch.empty_like(img_h).pin_memory(), torch.empty_like(txt_h).pin_memory()] for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        out_ready = [torch.cuda.Event() for _ in range(2)]
        out_free = [torch.cuda.Event() for _ in range(2)]
        graphs = None
        if not args.no_graph:
            graphs = []
            for b in range(2):
                for dst, src in zip(bufs[b], (img_d, txt_d, vec_d)):
                    dst.copy_(src)
                gf = GraphedForward(lambda i, t, v: block(i, t, v, pe_d), tuple(bufs[b]))
                bufs[b] = list(gf.static_inputs)  # the copies land directly in the captured inputs
                graphs.append(gf)

        def e2e_steps(n):
            keep = []
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(in_free[b])
                    for dst, src in zip(bufs[b], (img_h, txt_h, vec_h)):
                        dst.copy_(src, non_blocking=True)
                    in_ready[b].record(s_in)
                s_cmp.wait_event(in_ready[b])
                if graphs is not None:
                    s_cmp.wait_event(out_free[b])  # this graph's output buffers were read out
                    graphs[b].graph.replay()
                    oi, ot = graphs[b].static_outputs
                else:
                    oi, ot = block(bufs[b][0], bufs[b][1], bufs[b][2], pe_d)
                in_free[b].record(s_cmp)
                out_ready[b].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(out_ready[b])
                    outs_h[b][0].copy_(oi, non_blocking=True)
                    outs_h[b][1].copy_(ot, non_blocking=True)
                    out_free[b].record(s_out)
                    if graphs is None:
                        oi.record_stream(s_out)
                        ot.record_stream(s_out)
                keep.append((oi, ot))
                if len(keep) > 2:
                    keep.pop(0)
            s_cmp.wait_stream(s_out)

        for ev in out_free:
            ev.record(s_cmp)
        for ev in in_free:
            ev.record(s_cmp)
        e2e_steps(args.warmup)
        barrier()
        t0 = time.perf_counter()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        e2e_steps(args.steps)
        g1.record()
        barrier()
        e2e_ms = max_over_ranks(max(g0.elapsed_time(g1), 0.0))
        e2e_wall_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
        e2e_out_same = bool(torch.equal(outs_h[(args.steps - 1) & 1][0].float(), out_img_h))
        del graphs, bufs

        # ------------------------------------------------------------ sustained regime
        # The same captured step replayed for at least two seconds: long enough for the GPU to
        # settle at its power cap, which a run of some tens of steps does not reach.
        sustained = None
        if not args.no_extras and graphed is not None:
            n_sus = max(int(2.2 / (ms / args.steps * 1e-3)), 10)
            sus_sampler = ClockSampler(local_rank, period_s=0.02)
            sus_sampler.start()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n_sus):
                step()
            b.record()
            barrier()
            sus_ms = max_over_ranks(a.elapsed_time(b))
            sus_clocks = sus_sampler.stop()
            sustained = {"steps": n_sus, "seconds": sus_ms * 1e-3, "ms_per_step": sus_ms / n_sus,
                         "value": world * TOKENS * n_sus / (sus_ms * 1e-3), "unit": UNIT,
                         "block_tflops_achieved": BLOCK_FLOP * n_sus / (sus_ms * 1e-3) / 1e12, "clocks": sus_clocks}

    code, where = _lib.device_status()
    if code != 0:
        raise SystemExit(f"device status word reports error {code} at {where}")

    # ---------------------------------------------------------------- sub-records (all ranks take part)
    # A sub-record that fails must not take the headline line with it: its error is recorded in its
    # place, and the sub-records after it are skipped (after a failed collective the ranks may no
    # longer be in step).
    extras = {}
    extras_ok = True

    def guarded(name, fn):
        nonlocal extras_ok
        if not extras_ok:
            extras[name] = {"skipped": "an earlier sub-record failed"}
            return
        try:
            extras[name] = fn()
        except BaseException as e:  # noqa: BLE001
            if isinstance(e, KeyboardInterrupt):
                raise
            extras[name] = {"error": repr(e)[:400]}
            extras_ok = False

    if not args.no_extras:
        guarded("host_copy", lambda: host_copy_probe(dev, barrier, max_over_ranks))
        del block, graphed
        torch.cuda.empty_cache()

        def dit_record():
            dit = dit_measure(dev, min(args.steps, 20), min(args.warmup, 3), barrier=barrier, max_over_ranks=max_over_ranks)
            dit["tokens_per_s"] = world * dit["tokens_per_s_per_gpu"]
            dit["e2e"]["tokens_per_s"] = world * dit["e2e"]["tokens_per_s_per_gpu"]
            dit["parallelism"] = (f"batch data-parallel x{world}: one full DiT step per GPU per step" if world > 1
                                  else "single GPU")
            return dit

        guarded("dit", dit_record)
        if world > 1 and H % world == 0:
            # both exchanges; the record's own figures are those of the faster one, the other's
            # step time sits beside them
            def ulysses_record():
                recs = {ex: ulysses_measure(rank, local_rank, world, min(args.steps, 20), args.warmup, ex,
                                            single_rank_baseline=(ex == "peer"), no_graph=args.no_graph)
                        for ex in ("peer", "nccl")}
                single = recs["peer"]["single_gpu_ms_per_step"]
                for r in recs.values():
                    r["single_gpu_ms_per_step"] = single
                    r["efficiency_vs_single_gpu"] = single / (world * r["ms_per_step"])
                best = min(recs, key=lambda ex: recs[ex]["ms_per_step"])
                out = dict(recs[best])
                out["ms_per_step_by_exchange"] = {ex: r["ms_per_step"] for ex, r in recs.items()}
                out["efficiency_by_exchange"] = {ex: r["efficiency_vs_single_gpu"] for ex, r in recs.items()}
                for k in ("assembly_scatter_kernel_ms", "assembly_scatter_nvlink_gbs_per_gpu"):
                    if k in recs["peer"]:
                        out[k] = recs["peer"][k]
                return out

            guarded("ulysses", ulysses_record)

    # Peak for the roofline fraction: what cuBLAS delivers at the SM clock the timed launches ran at.
    # The driver measured cuBLAS twice: as a burst (best of ten launches) and in a seconds-long loop
    # at the power cap, for which it also recorded the median SM clock.  The loop figure per MHz,
    # times the median clock sampled over this run's launches, is the tensor rate cuBLAS would reach
    # at that clock; the burst figure caps it (a burst is power-limited too).  Near the maximum clock
    # this is the burst peak, deep in the power-capped regime it falls towards the loop figure.
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        pk = json.loads(peaks_path.read_text())
        burst, sustained_peak, src = pk["bf16_tflops"], pk["bf16_tflops_sustained"], "measured"
        sustained_clock = (pk.get("clocks_under_load") or {}).get("sm_mhz_median") or 1327.0
    else:
        burst, sustained_peak, sustained_clock, src = 1590.0, 1400.0, 1300.0, "fallback"
    sm_dom, sm_max = dom_clocks.get("sm_mhz"), dom_clocks.get("sm_max_mhz")
    if sm_dom is None:
        peak, regime = burst, "burst (no clock samples)"
    else:
        at_clock = sustained_peak * sm_dom / sustained_clock
        peak = min(burst, at_clock)
        regime = ("burst" if peak == burst else "sustained, scaled to the sampled clock") + \
                 f" (median SM clock over the timed launches {sm_dom} of {sm_max} MHz; the seconds-long cuBLAS loop ran at {sustained_clock} MHz)"
    dom_flop = 2.0 * DOM_M * DOM_N * DOM_K
    achieved = dom_flop / (dom_ms * 1e-3) / 1e12
    traffic, traffic_src = traffic_from_profile()

    if rank == 0:
        value = world * TOKENS * args.steps / (ms * 1e-3)
        e2e_value = world * TOKENS * args.steps / (e2e_ms * 1e-3)
        h2d = sum(t.numel() * t.element_size() for t in (img_h, txt_h, vec_h))
        d2h = sum(t.numel() * t.element_size() for t in (img_h, txt_h))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "parallelism": f"batch data-parallel x{world}" if world > 1 else "single GPU",
                "launch": "eager" if args.no_graph else "cuda graph replay of the module call",
                "l2": "no flush: 0.68 GB of weights + 0.3 GB of activations per step exceed the 126 MB L2",
                "block_tflop": BLOCK_FLOP / 1e12,
                "block_tflops_achieved": BLOCK_FLOP * args.steps / (ms * 1e-3) / 1e12,
                **extras,
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps, "wall_ms_per_step": e2e_wall_ms / args.steps,
                    "output_equals_device_resident_run": e2e_out_same},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {
                "bound": "tensor", "kernel": f"gemm_pair_kernel, grouped MLP-up M={L_TXT}+{L_IMG} K={DOM_K} N={DOM_N} +bias+GELU",
                "achieved": achieved, "peak": peak, "peak_source": f"{src} cuBLAS bf16, {regime}", "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_burst": burst, "peak_sustained": sustained_peak,
                "launch_ms": dom_ms, "launches_timed": len(durs), "launch_us_x_sm_mhz": (dom_ms * 1e3 * sm_dom) if sm_dom else None,
                "clocks": dom_clocks, "traffic": traffic, "traffic_source": traffic_src,
            },
        }
        if sustained is not None:
            line["sustained"] = sustained
        if not args.no_cpu_baseline:
            # The CPU oracle on this rank's inputs: its output is what the timed step's output is
            # checked against; at one GPU it is also timed as the CPU baseline.
            runs = 3 if world == 1 else 1
            t, threads, want = cpu_block_time(L_IMG, L_TXT, runs=runs, warm=1 if world == 1 else 0, seed=SEED + rank)
            line["parity"] = {"rel_l2_img": rel_l2(out_img_h, want[0]), "rel_l2_txt": rel_l2(out_txt_h, want[1]),
                              "bound": 1e-2, "against": "fp32 CPU oracle on the same bf16-rounded weights and inputs; "
                              "outputs of the last timed " + ("eager step" if args.no_graph else "graph replay")}
            if world == 1:
                line["cpu_baseline"] = {
                    "value": TOKENS / t, "unit": UNIT, "cores": threads, "kind": "port",
                    "sample": f"3 forward passes of the same double-stream block ({L_IMG}+{L_TXT} tokens, fp32, torch CPU)",
                }
        print(json.dumps(line), flush=True)
        if "parity" in line and max(line["parity"]["rel_l2_img"], line["parity"]["rel_l2_txt"]) > 1e-2:
            raise SystemExit("the timed step's outputs differ from the CPU oracle by more than 1e-2 relative L2")
    if world > 1:
        try:
            if extras_ok:
                dist.barrier()
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001  (a rank that failed a sub-record may already be gone)
            pass


if __name__ == "__main__":
    main()
