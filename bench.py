#!/usr/bin/env python3
"""Benchmark of the quantized-LLM hot path: Q4_0 decode tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at N=1: TinyLlama-1.1B architecture with
seeded random Q4_0 weights (f16 embeddings and norms), batch 1, 512-token
prompt, then greedy decode with an f16 KV cache.  A "step" is one decode step
(one token).  Prints ONE JSON line.

  value        tokens/s over K steps replayed back to back on the device
               (token ids, positions and the sampled token stay in HBM), CUDA
               events on the library's stream;
  e2e          the same K steps through the host-buffer entry point
               tlc_llama_decode_host: per step the token id goes up from pinned
               memory and the sampled token comes back, with a stream sync;
  roofline     the dominant kernel (the fused dequant-GEMV): algorithmic bytes
               per launch / its average launch duration, timed by replaying only
               the step's GEMV launches between two CUDA events;
  cpu_baseline the CPU oracle's restatement of the reference's literal CPU
               path (single thread, f16 running sum), on a bounded sample.

With --gpus N > 1 (launched under torchrun, one process per GPU) the workload is
Llama-2-70B-shape Q4_0 decode, tensor-parallel over the N GPUs with an NCCL all-reduce after the row-parallel projections (TinyLlama
has 4 KV heads and cannot be split 8 ways).  The line names that workload and
says scaling "strong"; it is a different workload from the N=1 line.
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
sys.path.insert(0, ROOT)

PROMPT_TOKENS = 512
SEED = 2
METRIC = "q4_0_decode_tokens_per_s"
L2_BYTES = 126 * 1000 * 1000


def workload_name(n_gpus: int, batch: int = 1, big: bool = False) -> str:
    """The `config.workload` string, the same in both arms (`--impl ours` / `--impl reference`)."""
    if n_gpus > 1 or big:
        return (f"llama-2-70b-shape q4_0 decode, TP{n_gpus}, batch {batch}, 2048-token context; "
                f"NOT the N=1 workload (tinyllama)")
    return "tinyllama-1.1b q4_0 decode, batch 1, 512-token prompt"


def profiled_traffic(key: str, algorithmic_bytes: float | None = None):
    """DRAM bytes per launch of a kernel from the ncu summaries under profiles/ (traffic.json):
    (bytes or None, where it comes from).  Taken from a capture, never measured in the run.  An
    entry holds either the captured bytes per launch of exactly this workload, or -- for workloads
    too large to capture -- the ratio of captured to algorithmic bytes of a smaller capture of the
    same kernel, applied to this run's algorithmic bytes per launch."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None, None
    entry = json.load(open(path)).get(key)
    if not entry:
        return None, None
    if "dram_bytes_per_launch" in entry:
        return float(entry["dram_bytes_per_launch"]), \
            f"from profiles/{entry['summary']} (one ncu capture), not measured in this run"
    if "ratio_to_algorithmic" in entry and algorithmic_bytes:
        return float(entry["ratio_to_algorithmic"]) * algorithmic_bytes, \
            (f"algorithmic bytes x {entry['ratio_to_algorithmic']} (DRAM / algorithmic bytes of the capture in "
             f"profiles/{entry['summary']}, a smaller case of the same kernel), not measured in this run")
    return None, None


def load_peaks() -> dict:
    """Measured roofline denominators (MEASURED_PEAKS.json beside this file), else the pool's fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def tinyllama_bytes_per_token(arch, context: int) -> int:
    """Algorithmic HBM bytes of one decode step: every Q4_0 weight once, norm weights, one
    embedding row, the KV cache of `context` tokens read and one position written."""
    d, qd, kvd, f = arch.d_model, arch.n_heads * arch.head_dim, arch.n_kv_heads * arch.head_dim, arch.ffn_dim
    q4 = lambda n, k: n * (k // 32) * 18
    layer = q4(qd, d) + 2 * q4(kvd, d) + q4(d, qd) + 2 * q4(f, d) + q4(d, f)
    weights = arch.n_layers * layer + q4(arch.vocab, d)
    norms = (2 * arch.n_layers + 1) * d * 2
    kv = arch.n_layers * 2 * kvd * 2 * (context + 1)
    return weights + norms + d * 2 + kv


def gemv_bytes_per_step(arch, m: int = 1) -> tuple[int, int]:
    """(algorithmic bytes, launches) of the GEMV launches of one decode step:
    N*(K/32)*18 + 2*M*K + 2*M*N per linear, summed per fused launch."""
    d, qd, kvd, f = arch.d_model, arch.n_heads * arch.head_dim, arch.n_kv_heads * arch.head_dim, arch.ffn_dim
    lin = lambda n, k: n * (k // 32) * 18 + 2 * m * n
    x = lambda k: 2 * m * k
    layer = (lin(qd, d) + 2 * lin(kvd, d) + x(d)) + (lin(d, qd) + x(qd)) + (2 * lin(f, d) + x(d)) + (lin(d, f) + x(f))
    return arch.n_layers * layer + lin(arch.vocab, d) + x(d), 4 * arch.n_layers + 1


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None
        self.t0, self.t1 = None, None

    def mark_start(self):
        """The timed region starts now (samples outside it are kept apart)."""
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows, window = [r for _, r in self.rows], "sampler lifetime"
        if self.t0 is not None and self.t1 is not None:
            # nvidia-smi reports about 0.1 s late: a sample belongs to the region it was taken in
            inside = [r for t, r in self.rows if self.t0 <= t - 0.05 <= self.t1 + 0.15]
            if inside:
                rows, window = inside, "timed region"
            else:
                window = "warm-up + timed region (the timed region is shorter than the sampling period)"
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def dist_setup(n_gpus: int):
    """Under torchrun: NCCL process group for the barrier and the max-over-ranks reduction."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


class CpuSample:
    """A bounded sample of the reference's CPU path for one decode token.

    Restated by oracle/tl_ref.c: GGUF dequantization (src/model/formats/gguf.rs:68-112) happens
    once at load upstream and is not timed; per token the linears run as transpose + matmul_cpu with
    an f16 running sum on one thread (src/ops/matmul.rs:201-228, :293-297).  One `step()` runs the
    seven linears of one layer plus `head_rows` lm_head rows; a token costs n_layers * layer +
    lm_head, so tokens/s = 1 / (n_layers * row_div * t_layer + vocab / head_rows * t_head).
    row_div > 1 takes only every row_div-th part of each linear's rows (the cost is linear in the
    rows) so that the 70B shape stays a bounded sample too.  Attention, norms and sampling are not
    charged to the CPU (that favours the CPU).
    """

    def __init__(self, arch, seed: int, row_div: int = 1, head_rows: int = 4000):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import tl_ref as ref
        from tensorlogic_b200 import synth
        self.ref, self.arch, self.row_div, self.head_rows = ref, arch, row_div, head_rows
        d, qd, kvd, f = arch.d_model, arch.n_heads * arch.head_dim, arch.n_kv_heads * arch.head_dim, arch.ffn_dim
        shapes = [("attn_q", qd, d), ("attn_k", kvd, d), ("attn_v", kvd, d), ("attn_output", d, qd), ("ffn_gate", f, d),
                  ("ffn_up", f, d), ("ffn_down", d, f)]
        self.ws = []
        for name, n, k in shapes:
            n = max(16, n // row_div)
            raw = synth.blocks(2, seed, synth.tensor_id(f"blk.0.{name}.weight"), n, k)
            self.ws.append((ref.dequant(2, raw, n * k).reshape(n, k), synth.activations(seed, f"cpu.{name}", (1, k))))
        raw = synth.blocks(2, seed, synth.tensor_id("output.weight"), head_rows, d)
        self.head = ref.dequant(2, raw, head_rows * d).reshape(head_rows, d)
        self.xh = synth.activations(seed, "cpu.head", (1, d))
        self.t_layer, self.t_head, self.reps = 0.0, 0.0, 0

    def step(self, count: bool = True) -> float:
        """One sample; returns its wall time in seconds."""
        t0 = time.perf_counter()
        for w, x in self.ws:
            self.ref.linear_literal(x, w)
        t1 = time.perf_counter()
        self.ref.linear_literal(self.xh, self.head)
        t2 = time.perf_counter()
        if count:
            self.t_layer += t1 - t0
            self.t_head += t2 - t1
            self.reps += 1
        return t2 - t0

    def token_seconds(self) -> float:
        a = self.arch
        return a.n_layers * (self.t_layer / self.reps) * self.row_div + (self.t_head / self.reps) * (a.vocab / self.head_rows)

    def sample_fraction(self) -> float:
        """Multiply-adds of one sample / multiply-adds of one token."""
        a = self.arch
        sample = sum(w.size for w, _ in self.ws) + self.head.size
        token = a.n_layers * sum(w.size for w, _ in self.ws) * self.row_div + a.vocab * a.d_model
        return sample / token

    def summary(self) -> dict:
        ref, a = self.ref, self.arch
        # the multi-threaded f32-accumulating variant (no counterpart upstream), for context
        t0 = time.perf_counter()
        for w, x in self.ws:
            ref.linear_f32acc(x, w)
        ref.linear_f32acc(self.xh, self.head)
        t_mt = time.perf_counter() - t0
        div = f", 1/{self.row_div} of their rows" if self.row_div > 1 else ""
        return {"value": 1.0 / self.token_seconds(), "unit": "tokens/s", "cores": 1, "kind": "port",
                "sample": (f"{self.reps}x (7 linears of one layer{div} + {self.head_rows} "
                           f"lm_head rows), literal f16-accumulate matmul on "
                           f"pre-dequantized f16 weights, scaled to {a.n_layers} layers + {a.vocab} lm_head rows; "
                           f"attention, norms and sampling not counted (favours the CPU)"),
                "sample_fraction_of_a_token": self.sample_fraction(),
                "f16c": bool(ref.uses_f16c()), "host_cores_available": os.cpu_count(),
                "mt_f32acc_tokens_per_s": self.sample_fraction() / t_mt, "mt_threads": ref.num_threads()}


def cpu_baseline(arch, seed: int, budget_s: float = 12.0, row_div: int = 1) -> dict:
    """The reference's CPU path on a bounded sample (CpuSample), repeated for about budget_s seconds."""
    sample = CpuSample(arch, seed, row_div)
    t_start = time.perf_counter()
    while sample.reps < 1 or (time.perf_counter() - t_start) < budget_s:
        sample.step()
    return sample.summary()


def run_reference(args, rank: int, world: int) -> None:
    """--impl reference: the reference's own CPU implementation of the path (no GPU work).

    A "step" of this arm is one bounded sample of a token's work (CpuSample.step); W samples warm
    up, K are timed.  `ms_per_step` is the measured time of a sample; `value` (tokens/s) is that
    time scaled to a whole token, and `extrapolation` says by how much."""
    if rank != 0:
        return
    from tensorlogic_b200.model import LLAMA2_70B, TINYLLAMA
    # the same workload as this repo's arm at that N: TinyLlama at N = 1, the 70B shape beyond
    big = args.gpus > 1 or args.workload == "decode70b"
    arch = LLAMA2_70B if big else TINYLLAMA
    t_wall = time.perf_counter()
    sample = CpuSample(arch, SEED, row_div=16 if big else 1)
    # a sample takes ~0.5 s: bound the run to a few minutes whatever K is asked for
    K = max(1, min(args.steps, 256))
    for _ in range(max(0, min(args.warmup, 8))):
        sample.step(count=False)
    t0 = time.perf_counter()
    for _ in range(K):
        sample.step()
        if time.perf_counter() - t0 > 150.0:
            break
    timed = time.perf_counter() - t0
    base = sample.summary()
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": sample.reps, "warmup": args.warmup, "ms_per_step": 1e3 * timed / sample.reps,
        "higher_is_better": True, "scaling": "strong" if big else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": workload_name(args.gpus, args.batch, big),
                   "note": "reference CPU path (transpose + f16-accumulating matmul_cpu, 1 thread; the reference has no "
                           "multi-GPU path: one host process); a step is a bounded sample of one token's linears",
                   "wall_s": round(time.perf_counter() - t_wall, 1)},
        "extrapolation": {"step_is": "one sample = 7 linears of one layer + 4000 lm_head rows" +
                                     (" (1/16 of the rows of each)" if big else ""),
                          "sample_fraction_of_a_token": base["sample_fraction_of_a_token"],
                          "seconds_per_token_extrapolated": 1.0 / base["value"],
                          "value_is": "1 / seconds_per_token_extrapolated"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, world: int, local: int) -> None:
    import torch
    from tensorlogic_b200.api import Device
    from tensorlogic_b200.model import TINYLLAMA, Llama, synthetic_model
    from tensorlogic_b200 import synth
    arch = TINYLLAMA
    K, W = args.steps, max(args.warmup, 3)
    dev = Device(local)
    model = synthetic_model(dev, arch, SEED)
    max_seq = PROMPT_TOKENS + 2 * K + 3 * W + 64
    llm = Llama(dev, model, arch, max_seq=max_seq, max_batch=1, max_prefill=PROMPT_TOKENS)
    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local))
    ids = synth.token_ids(SEED, f"prompt.{rank}", PROMPT_TOKENS, arch.vocab)

    def barrier():
        dev.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        import torch.distributed as dist
        t = torch.tensor([ms], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    first, _ = llm.prefill(ids, return_logits=False)

    # ---- device-resident decode: K graph replays between two events ----
    llm.decode_enqueue(1, W)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = dev.launch_count
    with ClockSampler(local) as clocks:
        llm.decode_enqueue(1, W)       # nvidia-smi needs a moment to start: keep the GPU in the same state meanwhile
        barrier()
        launches0 = dev.launch_count
        clocks.mark_start()
        e0.record(stream)
        llm.decode_enqueue(1, K)
        e1.record(stream)
        barrier()
        clocks.mark_end()
    ms = max_over_ranks(e0.elapsed_time(e1))
    gpu_launches = dev.launch_count - launches0
    tok_s = world * K / (ms / 1e3)
    _, pos = llm.read_state(1)
    context_mid = int(pos[0]) - K // 2

    # ---- end to end through host buffers ----
    tok = int(llm.read_state(1)[0][0])
    for _ in range(W):
        tok = int(llm.decode([tok])[0][0])
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = int(llm.decode([tok])[0][0])
    dev.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    e2e_tok_s = world * K / (e2e_ms / 1e3)

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 6650.0, "fallback"
    persistent = llm.launches(7) == 1
    if persistent:
        # ---- dominant kernel: the persistent decode-step kernel itself.  One launch ran the K
        # timed steps, so its duration is the timed region and its algorithmic bytes are K steps'.
        bytes_per_launch = float(tinyllama_bytes_per_token(arch, context_mid)) * K
        kernel_us = ms * 1e3
        kernel_name = "decode_step_kernel<Q4_0> (one launch = the K timed decode steps)"
        kernel_launches_per_step = 1.0 / K
        traffic, traffic_src = None, None
        tpath = os.path.join(ROOT, "profiles", "decode_step_traffic.json")
        if os.path.exists(tpath):
            # DRAM bytes per decode step from one ncu capture of a short run of this workload
            # (profiles/decode_step_kernel_tinyllama.md gives the command), scaled to K steps.
            t = json.load(open(tpath))
            traffic = float(t["dram_bytes_per_step"]) * K
            traffic_src = t.get("source", "ncu capture, see profiles/decode_step_kernel_tinyllama.md") + \
                "; not measured in this run, scaled by the steps per launch"
    else:
        # ---- dominant kernel: replay only the GEMV launches of a step ----
        llm.decode_enqueue(1, W, parts=1)
        dev.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        llm.decode_enqueue(1, K, parts=1)
        g1.record(stream)
        dev.synchronize()
        gemv_bytes, gemv_launches = gemv_bytes_per_step(arch)
        assert llm.launches(1) == gemv_launches, (llm.launches(1), gemv_launches)
        kernel_us = g0.elapsed_time(g1) * 1e3 / (K * gemv_launches)
        bytes_per_launch = gemv_bytes / gemv_launches
        kernel_name = "gemv_mma_kernel<Q4_0> (fused dequant-GEMV, M=1)"
        kernel_launches_per_step = gemv_launches
        traffic, traffic_src = profiled_traffic("tinyllama_decode_gemv")
    achieved = bytes_per_launch / (kernel_us * 1e-6) / 1e9
    step_bytes = tinyllama_bytes_per_token(arch, context_mid)

    if rank != 0:
        return
    base = cpu_baseline(arch, SEED) if world == 1 else None
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(1),
                   "context_tokens_mid_run": context_mid, "parallelism": "single" if world == 1 else f"replicas x{world}",
                   "l2": "weights of one step (582 MB) exceed the 126 MB L2: every step re-reads them from HBM",
                   "step_hbm_bytes": step_bytes, "step_hbm_gbs": step_bytes / (ms / K * 1e-3) / 1e9,
                   "launches_per_step": llm.launches(7) if not persistent else
                   f"one persistent cooperative launch runs all {K} timed steps (e2e: one launch per step)",
                   "seed": SEED},
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4,
                "ms_per_step": e2e_ms / K},
        "gpu_launches": int(gpu_launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": kernel_name,
                     "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                     "frac": achieved / peak, "bytes_per_launch": bytes_per_launch, "us_per_launch": kernel_us,
                     "launches_per_step": kernel_launches_per_step, "traffic": traffic,
                     "traffic_source": traffic_src},
    }
    if base is not None:
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)


def llama_bytes_per_step(arch, tp: int, batch: int, context: int) -> int:
    """Algorithmic HBM bytes one rank moves per decode step: its shard of every Q4_0 weight once,
    plus its KV heads' cache of `context` positions per sequence."""
    d, qd, kvd, f = arch.d_model, arch.n_heads * arch.head_dim, arch.n_kv_heads * arch.head_dim, arch.ffn_dim
    q4 = lambda n, k: n * (k // 32) * 18
    layer = q4(qd, d) + 2 * q4(kvd, d) + q4(d, qd) + 2 * q4(f, d) + q4(d, f)
    weights = (arch.n_layers * layer + q4(arch.vocab, d)) // tp
    kv = arch.n_layers * 2 * (kvd // tp) * 2 * (context + 1) * batch
    return weights + kv


def time_decode(dev, llm, stream, batch, K, W, barrier, clocks=None):
    """W warm-up steps, then K steps between two CUDA events on the library's stream: ms, launches."""
    import torch
    llm.decode_enqueue(batch, W)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = dev.launch_count
    if clocks:
        clocks.mark_start()
    e0.record(stream)
    llm.decode_enqueue(batch, K)
    e1.record(stream)
    barrier()
    if clocks:
        clocks.mark_end()
    return e0.elapsed_time(e1), dev.launch_count - launches0


def run_tp(args, rank: int, world: int, local: int) -> None:
    """Llama-2-70B-shape Q4_0 decode, tensor-parallel over the N GPUs of the
    launch (N = 1 with --workload decode70b: the whole 38.65 GB model on one GPU):
    column-parallel q/k/v/gate/up/lm_head, row-parallel o/down with an all-reduce after each (one
    peer-memory kernel fused with the residual add; NCCL with --nccl-allreduce), 2048 positions
    already in the KV cache (filled with random f16 on the device).  With N > 1, rank 0 also times
    the unsharded model on its own GPU afterwards, so that the line carries `speedup_vs_tp1`."""
    import torch
    from tensorlogic_b200.api import Device
    from tensorlogic_b200.model import LLAMA2_70B, Llama, synthetic_model
    arch, batch, context = LLAMA2_70B, args.batch, 2048
    shard_of = args.as_shard if world == 1 else 1
    if shard_of > 1:
        # One rank's share of the tensor-parallel model as a model of its own on one GPU: the same
        # kernels on the same shapes as a rank of TP<shard_of> runs, without the collectives
        # (the partial sums of o / down are simply used as they are).  Gives the compute floor of
        # a rank and a launch list that ncu can take (it must not wrap a multi-rank command).
        from tensorlogic_b200.model import LlamaArch
        arch = LlamaArch(arch.n_layers, arch.d_model, arch.n_heads // shard_of, arch.n_kv_heads // shard_of, arch.head_dim,
                         arch.ffn_dim // shard_of, arch.vocab // shard_of)
    K, W = args.steps, max(args.warmup, 3)
    dev = Device(local)
    comm = None
    if world > 1:
        import torch.distributed as dist
        from tensorlogic_b200.comm import Comm, unique_id
        box = [unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, device=torch.device("cuda", local))
        comm = Comm(dev, box[0], rank, world)
        if not args.nccl_allreduce:
            # peer-memory exchange: the [batch, d_model] all-reduces run as one kernel over NVLink
            def gather(blob):
                out = [None] * world
                dist.all_gather_object(out, blob)
                return out
            comm.enable_p2p(max(16, batch) * arch.d_model, gather)
    max_seq = context + 2 * K + 3 * W + 64
    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local))

    def barrier():
        dev.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def build(tp_rank, tp_size):
        model = synthetic_model(dev, arch, SEED, tp_rank=tp_rank, tp_size=tp_size, device_embeddings=True)
        llm = Llama(dev, model, arch, max_seq=max_seq, max_batch=batch, max_prefill=16, tp_rank=tp_rank, tp_size=tp_size)
        if tp_size > 1:
            llm.set_comm(comm)
        llm.fill_cache_random(SEED)
        llm.set_state([(7 + 13 * b) % arch.vocab for b in range(batch)], [context] * batch)
        return model, llm

    model, llm = build(rank, world)
    with ClockSampler(local) as clocks:
        llm.decode_enqueue(batch, W)   # nvidia-smi needs a moment to start
        ms, gpu_launches = time_decode(dev, llm, stream, batch, K, W, barrier, clocks)
    ms = max_over_ranks(ms)
    tok_s = batch * K / (ms / 1e3)

    # end to end: token ids up from the host, sampled tokens back, every step, on every rank
    toks = llm.read_state(batch)[0]
    for _ in range(W):
        toks = llm.decode(toks)[0]
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        toks = llm.decode(toks)[0]
    dev.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)

    # dominant kernel: the GEMV launches of a step, replayed alone (in a sharded model that
    # graph also holds the collectives that follow o/down and lm_head)
    llm.decode_enqueue(batch, W, parts=1)
    dev.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    llm.decode_enqueue(batch, K, parts=1)
    g1.record(stream)
    dev.synchronize()
    gemv_ms = max_over_ranks(g0.elapsed_time(g1))
    launches_per_step = llm.launches(7)

    # the one-GPU point of the scaling curve: the unsharded model on rank 0's GPU
    tp1 = None
    if world > 1 and not args.no_tp1:
        barrier()
        if rank == 0:
            del llm, model
            dev.pool_trim(0)
            K1 = min(K, 16)
            _m1, llm1 = build(0, 1)
            ms1, _ = time_decode(dev, llm1, stream, batch, K1, 3, lambda: dev.synchronize())
            tp1 = {"ms_per_step": ms1 / K1, "value": batch * K1 / (ms1 / 1e3), "steps": K1,
                   "note": "the whole model on rank 0's GPU, same batch and context, timed after the sharded run"}
            del llm1, _m1
        barrier()
    if rank != 0:
        return
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak, peak_src = (float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)") \
        if os.path.exists(peaks_path) else (6650.0, "fallback")
    d, qd, kvd, f = arch.d_model, arch.n_heads * arch.head_dim, arch.n_kv_heads * arch.head_dim, arch.ffn_dim
    q4 = lambda n, k: n * (k // 32) * 18
    wbytes = (arch.n_layers * (q4(qd, d) + 2 * q4(kvd, d) + q4(d, qd) + 2 * q4(f, d) + q4(d, f)) + q4(arch.vocab, d)) // world
    gemv_launches = 4 * arch.n_layers + 1
    us = gemv_ms * 1e3 / (K * gemv_launches)
    achieved = wbytes / gemv_launches / (us * 1e-6) / 1e9
    step_bytes = llama_bytes_per_step(arch, world, batch, context + 2 * W + K // 2)
    traffic, traffic_src = profiled_traffic(f"llama70b_tp{world if shard_of == 1 else shard_of}_gemv" if batch == 1 else "none",
                                            wbytes / gemv_launches)
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(world, batch, True) if shard_of == 1 else
                   f"ONE rank's share of llama-2-70b-shape q4_0 decode at TP{shard_of} (batch {batch}, 2048-token context) as "
                   f"a model of its own on one GPU, no collectives: the compute floor of a TP{shard_of} rank",
                   "parallelism": f"tp{world}" if shard_of == 1 else f"one shard of tp{shard_of}", "batch": batch,
                   "collectives_per_step": 2 * arch.n_layers + 1 if world > 1 else 0,
                   "allreduce_bytes": batch * d * 2 if world > 1 else 0,
                   "allreduce": ("one-shot peer-memory kernel fused with the residual add (data and sequence number in one "
                                 "8-byte store over NVLink, no fences)" if comm.p2p_ready
                                 else "nccl all-reduce + add kernel") if comm else "none (one GPU)",
                   "step_hbm_bytes_per_gpu": step_bytes,
                   "step_hbm_gbs_per_gpu": step_bytes / (ms / K * 1e-3) / 1e9,
                   "l2": "per-GPU weights (GBs) exceed the 126 MB L2", "launches_per_step": launches_per_step, "seed": SEED},
        "e2e": {"value": batch * K / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
                "d2h_bytes_per_step": 4 * batch, "ms_per_step": e2e_ms / K},
        "gpu_launches": int(gpu_launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "gemv_mma_kernel<Q4_0> (per-rank shard" +
                     ("; the time includes the collectives interleaved with the GEMV launches)" if world > 1 else ")"),
                     "achieved": achieved, "peak": peak,
                     "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                     "bytes_per_launch": wbytes / gemv_launches, "us_per_launch": us,
                     "launches_per_step": gemv_launches, "traffic": traffic, "traffic_source": traffic_src},
    }
    if tp1 is not None:
        line["tp1"] = tp1
        line["speedup_vs_tp1"] = tp1["ms_per_step"] / (ms / K)
    print(json.dumps(line), flush=True)


def run_kernel(args) -> None:
    """Micro-benchmark of one quantized linear (the profiling target): K launches of
    tlc_linear over weight copies that together exceed the L2, CUDA events on the
    library's stream.  m <= 16 runs the fused dequant-GEMV (HBM-bound: GB/s of
    algorithmic bytes), larger m the tcgen05 dequant-GEMM (tensor-bound: TFLOP/s)."""
    import torch
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import Device, QTensor
    qtype = {"q4_0": 2, "q8_0": 8}[args.qtype]
    n, k, m = args.n, args.k, args.m
    dev = Device(0)
    peaks = load_peaks()
    bb = 18 if qtype == 2 else 34
    w_bytes = n * (k // 32) * bb
    copies = max(1, min(64, -(-(2 * L2_BYTES) // w_bytes)))
    ws = [QTensor.synthetic(dev, qtype, n, k, SEED, 100 + i) for i in range(copies)]
    x = dev.tensor(synth.activations(SEED, "x", (m, k)))
    y = dev.empty((m, n))
    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", 0))
    lib = dev.lib

    def run(count):
        for i in range(count):
            rc = lib.tlc_linear(dev.handle, ws[i % copies].handle, x.ptr, m, k, y.ptr, None)
            if rc:
                raise RuntimeError(lib.tlc_last_error().decode())

    run(max(args.warmup, 1))
    dev.synchronize()
    l0 = dev.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        run(args.steps)
        e1.record(stream)
    dev.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    algo_bytes = w_bytes + 2 * m * k + 2 * m * n
    flops = 2.0 * m * n * k
    gemm = m > 16 and (dev.launch_count - l0) == args.steps and k % 64 == 0
    line = {"kernel": "linear", "qtype": args.qtype, "n": n, "k": k, "m": m, "launches": args.steps,
            "weight_copies": copies, "us_per_launch": us, "gpu_launches": dev.launch_count - l0}
    if m <= 16:
        line["roofline"] = {"bound": "hbm", "achieved": algo_bytes / us / 1e3, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": algo_bytes / us / 1e3 / peaks["hbm_gbs"], "peak_source": peaks["source"]}
    else:
        line["roofline"] = {"bound": "tensor", "achieved": flops / us / 1e6, "peak": peaks["bf16_tflops"],
                            "unit": "TFLOP/s", "frac": flops / us / 1e6 / peaks["bf16_tflops"],
                            "peak_source": peaks["source"], "path": "tcgen05 gemm" if gemm else "gemv passes"}
    print(json.dumps(line), flush=True)


def run_allreduce(args, rank: int, world: int, local: int) -> None:
    """--kernel allreduce under torchrun: the exchange step of the tensor-parallel decode on its
    own.  K x 100 back-to-back all-reduce + residual calls over --n f16 values (default 8192, the
    70B model's width) on every rank, CUDA events, max over ranks; the peer-memory kernel and the
    NCCL + add form side by side.  Says what one all-reduce costs when nothing else runs, i.e. how
    much of a tensor-parallel step is the exchange itself and how much is waiting for the slowest rank."""
    import torch
    import torch.distributed as dist
    from tensorlogic_b200.api import Device
    from tensorlogic_b200.comm import Comm, unique_id
    dev = Device(local)
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0, device=torch.device("cuda", local))
    comm = Comm(dev, box[0], rank, world)
    n = args.n if args.n != 28672 else 8192
    rng = np.random.default_rng(rank)
    part = dev.tensor(rng.standard_normal(n).astype(np.float16))
    res = dev.tensor(np.zeros(n, np.float16))
    out = dev.empty((n,))
    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local))
    lib = dev.lib

    def burst(count):
        for _ in range(count):
            rc = lib.tlc_allreduce_residual_f16(dev.handle, comm.handle, part.ptr, res.ptr, out.ptr, n)
            if rc:
                raise RuntimeError(lib.tlc_last_error().decode())

    def timed():
        burst(100 * max(args.warmup, 3))
        dev.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            burst(100 * args.steps)
            e1.record(stream)
        dev.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (100 * args.steps)], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    us_nccl = timed()

    def gather(blob):
        o = [None] * world
        dist.all_gather_object(o, blob)
        return o
    comm.enable_p2p(max(n, 16 * 8192), gather)
    us_p2p = timed()
    dev.set_option("comm_ll", 0)
    us_fenced = timed()
    dev.set_option("comm_ll", 1)
    if rank == 0:
        print(json.dumps({"kernel": "allreduce_residual", "n": n, "n_gpus": world, "calls": 100 * args.steps,
                          "us_per_call_peer_memory_flagged_words": us_p2p,
                          "us_per_call_peer_memory_fences_and_flags": us_fenced, "us_per_call_nccl_plus_add": us_nccl,
                          "note": "back-to-back calls from the host, nothing else on the stream; max over ranks"}),
              flush=True)
    dev.synchronize()
    comm.close()


def run_prefill(args, rank: int, world: int, local: int) -> None:
    """--workload prefill: Llama-2-7B-shape Q4_0 prefill of 2048 tokens.  The
    per-layer linears run as the tcgen05 dequant-GEMM; with N > 1 GPUs (torchrun) the weights are
    sharded column/row-parallel and the o / down partial sums are all-reduced (NCCL: 16 MB vectors).
    A step is one whole prefill; value = prompt tokens per second, roofline = tensor FLOP/s of the
    linears (2 * weights * tokens per step) against the measured bf16 peak."""
    import torch
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import Device
    from tensorlogic_b200.model import LLAMA2_7B, Llama, synthetic_model
    arch, tokens = LLAMA2_7B, 2048
    K, W = args.steps, max(args.warmup, 3)
    dev = Device(local)
    comm = None
    if world > 1:
        import torch.distributed as dist
        from tensorlogic_b200.comm import Comm, unique_id
        box = [unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, device=torch.device("cuda", local))
        comm = Comm(dev, box[0], rank, world)
    model = synthetic_model(dev, arch, SEED, tp_rank=rank if world > 1 else 0, tp_size=world, device_embeddings=True)
    llm = Llama(dev, model, arch, max_seq=tokens + 8, max_batch=1, max_prefill=tokens, tp_rank=rank if world > 1 else 0,
                tp_size=world)
    if comm is not None:
        llm.set_comm(comm)
    ids = synth.token_ids(SEED, "prefill.prompt", tokens, arch.vocab)
    stream = torch.cuda.ExternalStream(dev.stream, device=torch.device("cuda", local))

    def barrier():
        dev.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        llm.prefill(ids, return_logits=False)
    barrier()
    l0 = dev.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(K):
            llm.prefill(ids, return_logits=False)   # ids up, 2048-token forward, sampled token down
        e1.record(stream)
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank != 0:
        return
    peaks = load_peaks()
    weights = sum(r * c for n, (r, c) in arch.tensor_shapes().items()
                  if not n.endswith("norm.weight") and n not in ("token_embd.weight", "output.weight"))
    flops = 2.0 * weights * tokens  # lm_head runs for the last row only
    tflops = flops / (ms / K * 1e-3) / 1e12 / world
    line = {
        "metric": "q4_0_prefill_tokens_per_s", "value": tokens * K / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama-2-7b-shape q4_0 prefill, 2048 tokens, batch 1",
                   "parallelism": "single" if world == 1 else f"tp{world}",
                   "l2": "3.6 GB of weights per pass exceed the 126 MB L2", "seed": SEED},
        "e2e": {"value": tokens * K / (wall_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": tokens * 4,
                "d2h_bytes_per_step": 4, "ms_per_step": wall_ms / K},
        "gpu_launches": int(dev.launch_count - l0),
        "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<Q4_0> (dequant-GEMM of the layer linears)",
                     "achieved": tflops, "peak": peaks["bf16_tflops_sustained"], "peak_source": peaks["source"] +
                     " (sustained: the kernel runs inside a long step)", "unit": "TFLOP/s",
                     "frac": tflops / peaks["bf16_tflops_sustained"], "flops_per_step": flops, "traffic": None,
                     "note": "whole-step time: attention, norms, SiLU.mul and all-reduces are inside it"},
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "decode70b"],
                    help="decode: the headline workload (default); prefill: Llama-2-7B-shape 2048-token prefill; "
                         "decode70b: the Llama-2-70B-shape decode of the N > 1 runs on ONE GPU (the TP1 point)")
    ap.add_argument("--kernel", default=None, choices=["linear", "allreduce"],
                    help="micro-benchmark one kernel instead of the decode workload (see run_kernel)")
    ap.add_argument("--qtype", default="q4_0", choices=["q4_0", "q8_0"])
    ap.add_argument("--n", type=int, default=28672)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="decode batch of the tensor-parallel (N > 1) workload")
    ap.add_argument("--as-shard", type=int, default=1,
                    help="with --workload decode70b on one GPU: run ONE rank's share of TP<N> (no collectives)")
    ap.add_argument("--no-tp1", action="store_true",
                    help="N > 1: do not time the unsharded model on rank 0 afterwards (no `tp1` / `speedup_vs_tp1`)")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="N > 1: keep the all-reduces on NCCL instead of the peer-memory kernel (for comparison)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.kernel == "linear":
        run_kernel(args)
        return
    if world > 1:
        dist_setup(args.gpus)
    try:
        if args.kernel == "allreduce":
            if world < 2:
                raise SystemExit("--kernel allreduce needs torchrun with at least two ranks")
            run_allreduce(args, rank, world, local)
        elif args.workload == "prefill":
            run_prefill(args, rank, world, local)
        elif world > 1 or args.workload == "decode70b":
            run_tp(args, rank, world, local)
        else:
            run_ours(args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
