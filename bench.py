#!/usr/bin/env python
"""Benchmark of the two hot paths on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  The headline workload is the long-context attention forward
(B=2, H=32, S=16384, D=128, bf16, causal) per GPU: `value` is TFLOP/s summed over all ranks
(FLOPs = 4*B*H*S*S*D/2 per rank and step), timed with CUDA events over K launches with inputs
resident in HBM, max over ranks.  `e2e` is the same metric through the public Python call with
pinned HOST buffers: Q, K, V copied host->device and O device->host inside the timed region.
`also` carries the other configurations (attention at the GPT-2-small shape, the fused Lion
step on the GPT-2-medium list and, sharded ZeRO-1 style, on the Llama-7B list).
`cpu_baseline` times the CPU oracle (a C restatement of the reference's torch code) on a
bounded sample of the same workload.  `--impl reference` runs only that CPU arm.

Workloads: attn_c3 (default), attn_c2, attn_bwd_c3, lion_c4, lion_c5 (attn_prof, attn_short_prof and
attn_bwd_prof are the small shapes used for profiler captures).
Launch under torchrun for N > 1 (one rank per GPU); inputs are synthetic and seeded.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

ATTN = {
    # name: (B, H, S, D, causal)
    "attn_c2": (8, 12, 1024, 64, True),
    "attn_c3": (2, 32, 16384, 128, True),
    "attn_prof": (2, 32, 4096, 128, True),  # small case for profiler captures (inputs 201 MB > L2)
    "attn_short_prof": (32, 32, 1024, 128, True),  # the same for the one-tile-per-CTA kernel (805 MB)
}


def measured_traffic(name):
    """DRAM bytes per launch of the workload's kernel from the committed ncu summaries, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return float(json.load(f)[name]["dram_bytes_per_launch"])
    except Exception:
        return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---- clocks ------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the
    timed region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            try:  # NVML numbers GPUs without regard to CUDA_VISIBLE_DEVICES: match by UUID
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- distributed plumbing ------------------------------------------------------------------------

class Dist:
    def __init__(self, gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.on = self.world > 1
        if self.on:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # The one collective of this bench is a 13.5 GB all-gather that runs alone on the GPU:
            # with 64 channels NCCL moves it 5 to 10 % faster than with its default (measured on 2
            # and 4 GPUs of this pool: 640 against 577 and 687 against 654 GB/s bus bandwidth).
            os.environ.setdefault("NCCL_MIN_NCHANNELS", "64")
            os.environ.setdefault("NCCL_MAX_NCHANNELS", "64")
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        elif gpus > 1:
            raise SystemExit("launch with torchrun (one rank per GPU) for --gpus > 1")
        self.device = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.device)

    def barrier(self):
        if self.on:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_ms(self, ms: float) -> float:
        if not self.on:
            return ms
        t = torch.tensor([ms], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.on:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_steps(d: Dist, fn, steps: int, warmup: int, sampler=None):
    """W untimed steps, then exactly K steps between a barrier + synchronize on both sides;
    CUDA events on the launching (current) stream; returns the max over ranks of ms per step.
    Callers give `fn` inputs larger than L2, or several input sets that it uses in turn."""
    for _ in range(warmup):
        fn()
    d.barrier()
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    d.barrier()
    total = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    return d.max_ms(total) / steps, clocks


def graph_steps(d: Dist, fn, steps: int):
    """`steps` calls of fn captured into one CUDA graph on a side stream; returns the ms per step of
    one replay (CUDA events around it, max over ranks), after one untimed replay."""
    side = torch.cuda.Stream(device=d.device)
    side.wait_stream(torch.cuda.current_stream(d.device))
    graph = torch.cuda.CUDAGraph()
    keep = []
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(steps):
                keep.append(fn())  # outputs stay alive: every launch writes its own buffer, as in the eager loop
    torch.cuda.current_stream(d.device).wait_stream(side)
    graph.replay()
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    d.barrier()
    return d.max_ms(e0.elapsed_time(e1)) / steps


# ---- attention -------------------------------------------------------------------------------------

def attn_flops(B, H, S, D, causal):
    return 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)


def attn_inputs(B, H, S, D, device, seed):
    gen = torch.Generator(device=device).manual_seed(seed)
    return tuple(torch.randn(B, H, S, D, generator=gen, device=device, dtype=torch.float32).bfloat16()
                 for _ in range(3))


def attention_config(name: str, world: int, split: str):
    """The `config` object of an attention line (the GPU arm and the CPU reference arm print the same)."""
    B, H, S, D, causal = ATTN[name]
    strong = split == "strong" and world > 1
    heads = B * H // world if strong else B * H
    where = (f"the {B * H} (batch, head) pairs split {heads} per GPU over {world} GPUs" if strong else "per GPU")
    input_bytes = 3 * heads * S * D * 2
    sets = rotating_sets(input_bytes)
    return {"workload": f"{name}: attention fwd B={B} H={H} S={S} D={D} bf16 causal={causal}, {where}",
            "global_batch": B if strong else B * world,
            "l2": ("%d input sets used in turn (%.0f MB in total, larger than L2), no flush" % (sets, sets * input_bytes / 1e6)
                   if sets > 1 else "inputs (%.0f MB) larger than L2, no flush" % (input_bytes / 1e6))}


def rotating_sets(input_bytes: float) -> int:
    """How many distinct input sets a timed loop cycles through so that a set has left L2 (126 MB)
    before it is read again: one when a single set is already larger than twice L2, else enough
    sets for three times L2 between two uses of the same one."""
    if input_bytes > 2 * 126e6:
        return 1
    return int(-(-3 * 126e6 // input_bytes)) + 1


def bench_attention(d: Dist, name: str, steps: int, warmup: int, peaks, with_e2e=True, with_clocks=True,
                    split="weak"):
    """Forward of one attention workload.  split="weak": every rank runs the whole (B, H) shape on
    its own inputs.  split="strong": the B*H (batch, head) pairs of the ONE configured shape are
    divided over the ranks, rank r taking pairs [r*B*H/N, (r+1)*B*H/N) (pairs are independent:
    fast_ops/flash_attention/flash_attention_fwd.cu:57-59 indexes its grid by them), no collective;
    `value` is then the shape's FLOPs over the slowest rank's time."""
    import fast_ops_b200._lib as L
    from fast_ops_b200.flash_attention import flash_attention_forward

    B, H, S, D, causal = ATTN[name]
    flops_shape = attn_flops(B, H, S, D, causal)
    if split == "strong" and d.world > 1:
        if (B * H) % d.world:
            raise SystemExit(f"{B * H} (batch, head) pairs do not divide over {d.world} ranks")
        Bl, Hl = 1, B * H // d.world  # this rank's pairs, as heads of one batch entry
        flops_rank, flops_job = flops_shape / d.world, flops_shape
    else:
        split = "weak"
        Bl, Hl = B, H
        flops_rank, flops_job = flops_shape, flops_shape * d.world
    q, k, v = attn_inputs(Bl, Hl, S, D, d.device, seed=1000 + d.rank)
    lib = L.load()
    # a shape smaller than L2 is timed on several input sets used in turn, back to back like the
    # large ones, so that every launch reads its inputs from HBM
    sets = [(q, k, v)]
    for i in range(1, rotating_sets(3 * q.numel() * 2)):
        sets.append(attn_inputs(Bl, Hl, S, D, d.device, seed=1000 + d.rank + 100 * i))
    turn = [0]

    def fn():
        a, b, c = sets[turn[0] % len(sets)]
        turn[0] += 1
        return flash_attention_forward(a, b, c, causal=causal)

    launches0 = lib.fo_launch_count()
    sampler = ClockSampler(d.local_rank) if with_clocks else None
    ms, clocks = timed_steps(d, fn, steps, warmup, sampler)
    graphed = False
    if len(sets) > 1 and ms < 0.2:
        # a step this short is bound by the host's call path (about 17 us of Python and ctypes per
        # call, 40 us in this loop), which a training loop hides with a CUDA graph: time the same
        # K launches replayed from one
        launches0 = lib.fo_launch_count() - warmup
        ms = graph_steps(d, fn, steps)
        graphed = True
    del sets
    launches = (lib.fo_launch_count() - launches0 - warmup)
    if L.device_status(d.local_rank) != 0:
        raise RuntimeError("an attention kernel reported a timed-out wait")
    tflops_rank = flops_rank / (ms * 1e-3) / 1e12
    out = {
        "value": flops_job / (ms * 1e-3) / 1e12, "ms_per_step": ms, "gpu_launches": launches, "clocks": clocks,
        "scaling": split,
        "roofline": {"bound": "tensor", "achieved": tflops_rank, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tflops_rank / peaks["bf16_tflops"], "traffic": measured_traffic(name),
                     "peak_source": peaks["source"] + " cuBLAS bf16 burst",
                     "frac_of_sustained": tflops_rank / peaks["bf16_tflops_sustained"]},
        "config": attention_config(name, d.world, split),
    }
    if graphed:
        out["config"]["launch"] = "%d launches captured in one CUDA graph, the replay timed" % steps
    if with_e2e:
        # public call on HOST buffers: H2D of Q, K, V, forward, D2H of O, every step (the host
        # entry point pipelines the three over chunks of heads)
        from fast_ops_b200.flash_attention import flash_attention_forward_host

        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        ho = torch.empty_like(hq).pin_memory()
        del q, k, v
        torch.cuda.empty_cache()
        q = k = v = None

        def e2e_step():
            flash_attention_forward_host(hq, hk, hv, device=d.device, out=ho, causal=causal)

        e2e_steps = max(2, min(steps, 5))
        ms_e2e, _ = timed_steps(d, e2e_step, e2e_steps, 1)
        out["e2e"] = {"value": flops_job / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "h2d_bytes_per_step": 3 * hq.numel() * 2, "d2h_bytes_per_step": ho.numel() * 2,
                      "ms_per_step": ms_e2e, "steps": e2e_steps}
    return out


def bench_attention_bwd(d: Dist, name: str, steps: int, warmup: int, peaks):
    """Backward of the same attention shape: dQ, dK, dV from dO (three launches per step: delta,
    the main kernel, the rounding of dQ).  FLOPs = 2.5 x the forward's (five matmuls against two)."""
    import fast_ops_b200._lib as L
    from fast_ops_b200.flash_attention import flash_attention_backward, flash_attention_forward

    B, H, S, D, causal = ATTN[name]
    q, k, v = attn_inputs(B, H, S, D, d.device, seed=2000 + d.rank)
    dout = attn_inputs(B, H, S, D, d.device, seed=3000 + d.rank)[0]
    o, lse = flash_attention_forward(q, k, v, causal=causal, return_lse=True)
    lib = L.load()
    l0 = lib.fo_launch_count()
    ms, _ = timed_steps(d, lambda: flash_attention_backward(dout, q, k, v, o, lse, causal=causal), steps, warmup)
    launches = lib.fo_launch_count() - l0 - 3 * warmup
    if L.device_status(d.local_rank) != 0:
        raise RuntimeError("an attention kernel reported a timed-out wait")
    flops = 2.5 * attn_flops(B, H, S, D, causal)
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": f"{name} backward: dQ, dK, dV for B={B} H={H} S={S} D={D} bf16 causal={causal}, per GPU",
            "value": tf * d.world, "unit": "TFLOP/s", "ms_per_step": ms, "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "traffic": None,
                         "peak_source": peaks["source"] + " cuBLAS bf16 burst"}}


def bench_attention_variants(d: Dist, name: str, steps: int, warmup: int, peaks):
    """Forward and backward of the same shape with a per-head key bias (ALiBi-like, fp32, shape
    (1, H, 1, S)) and with dropout p = 0.17: TFLOP/s per GPU, the plain kernels' FLOP count."""
    import fast_ops_b200._lib as L
    from fast_ops_b200.flash_attention import flash_attention_backward, flash_attention_forward

    B, H, S, D, causal = ATTN[name]
    q, k, v = attn_inputs(B, H, S, D, d.device, seed=4000 + d.rank)
    dout = attn_inputs(B, H, S, D, d.device, seed=5000 + d.rank)[0]
    gen = torch.Generator(device=d.device).manual_seed(6000 + d.rank)
    bias = torch.randn(1, H, 1, S, generator=gen, device=d.device, dtype=torch.float32)
    flops = attn_flops(B, H, S, D, causal)
    out = {"workload": f"{name} with bias (1,H,1,S) fp32 / dropout 0.17: B={B} H={H} S={S} D={D} bf16 causal={causal}",
           "unit": "TFLOP/s per GPU"}
    for label, kw in (("bias", {"bias": bias}), ("dropout", {"dropout_p": 0.17, "rng": (0, 0)})):
        ms_f, _ = timed_steps(d, lambda: flash_attention_forward(q, k, v, causal=causal, **kw), steps, warmup)
        o, lse = flash_attention_forward(q, k, v, causal=causal, return_lse=True, **kw)
        ms_b, _ = timed_steps(d, lambda: flash_attention_backward(dout, q, k, v, o, lse, causal=causal, **kw),
                              steps, warmup)
        out[label] = {"fwd": flops / (ms_f * 1e-3) / 1e12, "fwd_ms": ms_f,
                      "bwd": 2.5 * flops / (ms_b * 1e-3) / 1e12, "bwd_ms": ms_b}
    if L.device_status(d.local_rank) != 0:
        raise RuntimeError("an attention kernel reported a timed-out wait")
    return out


def bench_attention_sweep(d: Dist, steps: int, warmup: int, peaks):
    """The metric's sweep: bf16 causal forward, H=32, D=128, batch x sequence = 32768 tokens, so that
    every point reads the same 805 MB (larger than L2): TFLOP/s per GPU by sequence length.  Every
    point carries the median SM clock sampled while it ran, so that points taken at different
    clocks (the power cap moves them) can be compared as time x MHz."""
    from fast_ops_b200.flash_attention import flash_attention_forward

    out = {"workload": "attention fwd bf16 causal, H=32 D=128, B*S=32768 tokens per GPU", "unit": "TFLOP/s per GPU"}
    for S in (1024, 2048, 4096, 8192, 16384):
        B = 32768 // S
        q, k, v = attn_inputs(B, 32, S, 128, d.device, seed=7000 + S + d.rank)
        sampler = ClockSampler(d.local_rank, period_s=0.002)
        ms, clocks = timed_steps(d, lambda: flash_attention_forward(q, k, v, causal=True), steps, warmup, sampler)
        tf = attn_flops(B, 32, S, 128, True) / (ms * 1e-3) / 1e12
        out[f"S{S}"] = {"value": tf, "ms_per_step": ms, "frac": tf / peaks["bf16_tflops"],
                        "sm_mhz": clocks["sm_mhz"], "reasons": clocks["reasons"]}
        del q, k, v
    return out


# A100 figures the reference publishes (wall-clock microseconds): fast_ops/lion/README.md:32-35
# ("ours" column) and fast_ops/flash_attention/README.md:80-97 (Triton forward, bf16, (1,12,S,128)).
PUBLISHED_A100_US = {
    "lion_8192_f16": 25.1, "lion_8192_bf16": 25.0, "lion_67108864_f16": 651.9, "lion_67108864_bf16": 710.1,
    "attn_S2048_full": 258.2, "attn_S2048_causal": 188.7, "attn_S4096_full": 926.5, "attn_S4096_causal": 548.9,
    "attn_S8192_full": 3415.7, "attn_S8192_causal": 1788.7,
}


def bench_reference_points(d: Dist):
    """The reference's own benchmark points, timed the way its scripts time them: wall clock of
    the public call with torch.utils.benchmark (which synchronises the device around the timed
    statement), median of a blocked autorange.  Lion: `lion.step()` on one tensor of 8192 and
    8192^2 elements, fp16 and bf16 (benchmarks/benchmark_lion.py:11-37).  Attention: forward of
    (batch 1, 12 heads, S, head_dim 128) bf16 in (B, S, H, D) layout, S in 2048/4096/8192, causal and
    not (benchmarks/benchmark_flash_attention.py:90; fast_ops/flash_attention/README.md:67-97)."""
    from torch.utils.benchmark import Timer

    from fast_ops.flash_attention.flash_attention_triton import flash_attn_triton
    from fast_ops.lion.lion_optimizer import Lion

    out = {"method": "torch.utils.benchmark.Timer.blocked_autorange median, wall clock of the public call",
           "unit": "us", "published": "A100 wall-clock figures from the reference's READMEs"}
    with torch.cuda.device(d.device):
        for size in (8192, 8192 ** 2):
            for dtype, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
                params = [torch.randn(size, dtype=dtype, device=d.device)]
                params[0].grad = torch.randn_like(params[0])
                lion = Lion(params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.1)
                lion.step()
                m = Timer(stmt="lion.step()", globals={"lion": lion}).blocked_autorange(min_run_time=0.3)
                us = m.median * 1e6
                key = f"lion_{size}_{tag}"
                out[key] = {"us": us, "a100_us": PUBLISHED_A100_US[key], "speedup_vs_a100": PUBLISHED_A100_US[key] / us,
                            "gbs": size * 10 / (us * 1e-6) / 1e9}
                del params, lion
        for S in (2048, 4096, 8192):
            q, k, v = (torch.randn(1, S, 12, 128, dtype=torch.bfloat16, device=d.device) for _ in range(3))
            for causal, tag in ((False, "full"), (True, "causal")):
                with torch.no_grad():
                    flash_attn_triton(q, k, v, None, causal)
                    m = Timer(stmt="f(q, k, v, None, causal)",
                              globals={"f": flash_attn_triton, "q": q, "k": k, "v": v, "causal": causal}
                              ).blocked_autorange(min_run_time=0.3)
                us = m.median * 1e6
                key = f"attn_S{S}_{tag}"
                flops = attn_flops(1, 12, S, 128, causal)
                out[key] = {"us": us, "a100_us": PUBLISHED_A100_US[key], "speedup_vs_a100": PUBLISHED_A100_US[key] / us,
                            "tflops": flops / (us * 1e-6) / 1e12}
            del q, k, v
        # what one call costs on the host when the kernel is negligible (one 128-row tile)
        q = torch.randn(1, 1, 128, 64, dtype=torch.bfloat16, device=d.device)
        from fast_ops_b200.flash_attention import flash_attention_forward

        m = Timer(stmt="f(q, q, q, causal=True)", globals={"f": flash_attention_forward, "q": q}
                  ).blocked_autorange(min_run_time=0.3)
        out["attention_call_floor_us"] = m.median * 1e6
    return out


def cpu_attention_sample(name: str, row_stride: int, reps: int):
    """Times the CPU oracle on one (batch, head) slice of the workload, every `row_stride`-th
    query row (the causal row costs are sampled evenly), all host threads."""
    import oracle

    B, H, S, D, causal = ATTN[name]
    gen = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 1, S, D, generator=gen).bfloat16() for _ in range(3))
    rows = range(0, S, row_stride)
    flops = sum(4.0 * D * ((r + 1) if causal else S) for r in rows)
    oracle.attention_fwd(q, k, v, causal=causal, row_range=(0, S, row_stride * 4))  # warm-up
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.attention_fwd(q, k, v, causal=causal, row_range=(0, S, row_stride))
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{name}: one (batch, head) slice, every {row_stride}th query row "
                      f"({flops / 1e9:.1f} GFLOP per run, median of {reps} runs of {t:.2f} s)"}, t


# ---- Lion ------------------------------------------------------------------------------------------

def gpt2_medium_shapes():
    shapes = [(50257, 1024), (1024, 1024)]
    for _ in range(24):
        shapes += [(1024, 3072), (3072,), (1024, 1024), (1024,), (1024, 4096), (4096,), (4096, 1024), (1024,),
                   (1024,), (1024,), (1024,), (1024,)]
    return shapes


def llama7b_shapes():
    shapes = [(32000, 4096), (32000, 4096)]
    for _ in range(32):
        shapes += [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)] + [(4096,)] * 2
    return shapes


def numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def bench_lion_c4(d: Dist, steps: int, warmup: int, peaks, with_e2e=True):
    """GPT-2-medium list: fp32 params/grads ~N(0,0.02)/N(0,1e-3), bf16 momentum, one launch per
    step; 16 algorithmic bytes per parameter."""
    import fast_ops_b200._lib as L
    from fast_ops_b200.lion import Lion

    gen = torch.Generator(device=d.device).manual_seed(7 + d.rank)
    shapes = gpt2_medium_shapes()
    params = [(torch.randn(s, generator=gen, device=d.device) * 0.02).requires_grad_(True) for s in shapes]
    for p in params:
        p.grad = torch.randn(p.shape, generator=gen, device=d.device) * 1e-3
    opt = Lion(params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.1, momentum_dtype=torch.bfloat16)
    n = sum(numel(s) for s in shapes)
    lib = L.load()
    l0 = lib.fo_launch_count()
    ms, _ = timed_steps(d, opt.step, steps, warmup)
    launches = lib.fo_launch_count() - l0 - warmup
    gbs = n * 16 / (ms * 1e-3) / 1e9
    # end to end: gradients arrive from pinned host memory, a parameter checksum goes back
    hg = [p.grad.cpu().pin_memory() for p in params]
    hres = torch.zeros(1).pin_memory()

    def e2e_step():
        for p, g in zip(params, hg):
            p.grad.copy_(g, non_blocking=True)
        opt.step()
        hres.copy_(params[-1].detach().sum().reshape(1), non_blocking=True)

    ms_e2e = timed_steps(d, e2e_step, 3, 1)[0] if with_e2e else float("nan")
    res = {"workload": f"lion_c4: GPT-2-medium list, {len(shapes)} tensors, {n} params, fp32 p/g, bf16 m, per GPU",
           "value": gbs * d.world, "unit": "GB/s", "ms_per_step": ms, "gpu_launches": launches,
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "traffic": measured_traffic("lion_c4"),
                        "peak_source": peaks["source"] + " copy"},
           "e2e": {"value": n * 16 / (ms_e2e * 1e-3) / 1e9 * d.world, "unit": "GB/s",
                   "h2d_bytes_per_step": n * 4, "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e}}
    del params, opt, hg
    torch.cuda.empty_cache()
    return res


def buffer_hash(t):
    """Position-weighted 64-bit checksum of a 16-bit tensor's bit patterns (wraps modulo 2^64),
    computed on its device in bounded pieces."""
    bits = t.view(torch.int16)
    piece = 1 << 26
    w = (torch.arange(piece, device=t.device, dtype=torch.int64) % 65521) + 1
    acc = torch.zeros((), device=t.device, dtype=torch.int64)
    for off in range(0, bits.numel(), piece):
        m = min(piece, bits.numel() - off)
        acc = acc * 31 + (bits[off:off + m].to(torch.int64) * w[:m]).sum()
    return acc


def zero1_parity_check(d: Dist, flat_p, flat_g, m_shard, begin, end, step_fn, hyper):
    """Runs ONE more ZeRO-1 step (outside any timed region) and checks it: a 2^20-element window in
    the middle of this rank's shard must equal the CPU oracle's step on the window's previous
    contents, bit for bit, and afterwards every rank must hold the same flat parameter buffer
    (checksums agree).  Returns "ok", or a description of the failure: it never raises, so that a
    rank does not leave while peers still have its memory mapped; main() turns a failure into a
    non-zero exit after the process group has been shut down."""
    import oracle

    lr, betas, wd = hyper
    w = min(1 << 20, end - begin)
    a = begin + ((end - begin - w) // 2) // 8 * 8
    p0, g0 = flat_p[a:a + w].cpu(), flat_g[a:a + w].cpu()
    m0 = m_shard[a - begin:a - begin + w].cpu()
    step_fn()
    torch.cuda.synchronize()
    oracle.lion_step(p0, g0, m0, lr, betas, wd)
    bad = 0
    if not torch.equal(flat_p[a:a + w].cpu(), p0):
        bad |= 1
    if not torch.equal(m_shard[a - begin:a - begin + w].cpu(), m0):
        bad |= 2
    if d.on:
        h = buffer_hash(flat_p)
        lo, hi = h.clone(), h.clone()
        d.dist.all_reduce(lo, op=d.dist.ReduceOp.MIN)
        d.dist.all_reduce(hi, op=d.dist.ReduceOp.MAX)
        if int(lo.item()) != int(hi.item()):
            bad |= 4
        flags = torch.tensor([bad & 1, bad & 2, bad & 4], device=d.device)  # NCCL has no bitwise OR: MAX per bit
        d.dist.all_reduce(flags, op=d.dist.ReduceOp.MAX)
        bad = int(flags.sum().item())
    if bad == 0:
        return "ok"
    what = [name for bit, name in ((1, "parameters differ from the oracle"), (2, "momentum differs from the oracle"),
                                   (4, "the ranks' flat buffers differ")) if bad & bit]
    return "FAILED: " + "; ".join(what)


def bench_lion_c5(d: Dist, steps: int, warmup: int, peaks):
    """Llama-7B list, bf16 p/g/m, 10 algorithmic bytes per parameter, ZeRO-1: each rank updates
    1/N of one flat buffer, then ONE NCCL all-gather of the updated bf16 weights.  Total work is
    fixed as N grows.  After the timed loops one more step is checked against the oracle and
    across the ranks (`parity_check`)."""
    import fast_ops_b200._lib as L
    from fast_ops_b200.lion import FlatLayout
    from fast_ops_b200.lion.lion_optimizer import _flat_step

    shapes = llama7b_shapes()
    layout = FlatLayout.build([numel(s) for s in shapes], d.world)
    n = sum(numel(s) for s in shapes)
    total = layout.total
    gen = torch.Generator(device=d.device).manual_seed(11)  # the same on every rank: replicas start equal
    flat_p = torch.empty(total, device=d.device, dtype=torch.bfloat16)
    flat_g = torch.empty(total, device=d.device, dtype=torch.bfloat16)
    piece = 1 << 28
    for off in range(0, total, piece):  # bounded temporaries
        m = min(piece, total - off)
        flat_p[off:off + m] = (torch.randn(m, generator=gen, device=d.device) * 0.02).bfloat16()
        flat_g[off:off + m] = (torch.randn(m, generator=gen, device=d.device) * 1e-3).bfloat16()
    begin, end = layout.shard_range(d.rank)
    m_shard = torch.zeros(end - begin, device=d.device, dtype=torch.bfloat16)
    lib = L.load()
    hyper = (3e-5, (0.9, 0.99), 0.1)

    def step_kernel():
        _flat_step(flat_p, flat_g, m_shard, begin, end, *hyper)

    def gather():
        if d.on:
            d.dist.all_gather_into_tensor(flat_p, flat_p[begin:end])

    def full_step():
        step_kernel()
        gather()

    l0 = lib.fo_launch_count()
    ms_full, _ = timed_steps(d, full_step, steps, warmup)
    launches = lib.fo_launch_count() - l0 - warmup
    ms_kernel, _ = timed_steps(d, step_kernel, steps, 1)
    ms_gather = timed_steps(d, gather, steps, 1)[0] if d.on else 0.0
    parity = zero1_parity_check(d, flat_p, flat_g, m_shard, begin, end, full_step, hyper)
    shard_bytes = (end - begin) * 10
    res = {"workload": f"lion_c5: Llama-7B list, {len(shapes)} tensors, {n} params, bf16 p/g/m, ZeRO-1 over "
                       f"{d.world} GPU(s) + all-gather of bf16 weights",
           "scaling": "strong",
           "value": n * 10 / (ms_full * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_full, "gpu_launches": launches,
           "kernel_ms": ms_kernel, "kernel_gbs_per_gpu": shard_bytes / (ms_kernel * 1e-3) / 1e9,
           "parity_check": parity,
           "roofline": {"bound": "hbm", "achieved": shard_bytes / (ms_kernel * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                        "unit": "GB/s", "frac": shard_bytes / (ms_kernel * 1e-3) / 1e9 / peaks["hbm_gbs"],
                        "traffic": measured_traffic("lion_c5") if not d.on else None,
                        "peak_source": peaks["source"] + " copy"}}
    if d.on:
        recv = (d.world - 1) / d.world * total * 2
        res["all_gather"] = {"ms": ms_gather, "bus_gbs": recv / (ms_gather * 1e-3) / 1e9,
                             "nccl_channels": os.environ.get("NCCL_MIN_NCHANNELS"),
                             "bytes_received_per_gpu": recv}
        # the same step with the distribution fused into the kernel: peer stores over NVLink into a
        # symmetric-memory flat buffer, ranks ordered by device-side barriers before and after
        try:
            import torch.distributed._symmetric_memory as symm_mem
            from fast_ops_b200.lion.lion_optimizer import _flat_step_push

            sym_p = symm_mem.empty(total, dtype=torch.bfloat16, device=d.device)
            sym_p.copy_(flat_p)
            del flat_p
            flat_p = sym_p
            hdl = symm_mem.rendezvous(sym_p, d.dist.group.WORLD)
            peers = [int(ptr) for r, ptr in enumerate(hdl.buffer_ptrs) if r != d.rank]

            def fused_step():
                hdl.barrier(channel=0)
                _flat_step_push(sym_p, flat_g, m_shard, begin, end, peers, *hyper)
                hdl.barrier(channel=1)

            ms_fused, _ = timed_steps(d, fused_step, steps, warmup)
            res["fused_gather"] = {"ms_per_step": ms_fused, "value": n * 10 / (ms_fused * 1e-3) / 1e9, "unit": "GB/s",
                                   "nvlink_egress_gbs_per_gpu": recv / (ms_fused * 1e-3) / 1e9,
                                   "speedup_vs_step_plus_all_gather": ms_full / ms_fused,
                                   "parity_check": zero1_parity_check(d, sym_p, flat_g, m_shard, begin, end,
                                                                      fused_step, hyper)}
        except Exception as exc:  # symmetric memory unavailable: report, keep the NCCL numbers
            res["fused_gather"] = {"unavailable": repr(exc)[:200]}
    del flat_p, flat_g, m_shard
    torch.cuda.empty_cache()
    return res


def cpu_lion_sample(reps: int):
    """Times the CPU oracle's Lion step on the first tensor of the GPT-2-medium list (wte)."""
    import oracle

    n = 50257 * 1024
    gen = torch.Generator().manual_seed(2)
    p = torch.randn(n, generator=gen) * 0.02
    g = torch.randn(n, generator=gen) * 1e-3
    m = torch.zeros(n, dtype=torch.bfloat16)
    oracle.lion_step(p, g, m, 1e-4, (0.9, 0.99), 0.1)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.lion_step(p, g, m, 1e-4, (0.9, 0.99), 0.1)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {"value": n * 16 / t / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"lion_c4: the 50257x1024 embedding only ({n} params), median of {reps} steps of {t:.3f} s"}


# ---- main ------------------------------------------------------------------------------------------

def run_reference_arm(args):
    """CPU arm: the oracle (a C port of the reference's torch code) on the host cores, on a
    bounded sample of the workload per step.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    name = args.workload
    if name.startswith("attn"):
        stride = 4 if name == "attn_c3" else 1
        cpu, _ = cpu_attention_sample(name, stride, max(1, args.steps))
        split = "strong" if (name == "attn_c3" and args.gpus > 1) else "weak"
        config = attention_config(name, args.gpus, split)
        metric, unit = "attention_fwd_tflops", "TFLOP/s"
    else:
        cpu = cpu_lion_sample(max(1, args.steps))
        config, metric, unit, split = {"workload": name}, "lion_step_hbm_gbs", "GB/s", "weak"
    line = {"impl": "reference", "metric": metric, "value": cpu["value"], "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": split,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="attn_c3",
                    choices=["attn_c3", "attn_c2", "attn_prof", "attn_short_prof", "attn_bwd_c3", "attn_bwd_prof", "lion_c4", "lion_c5"])
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-also", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")

    peaks = load_peaks()
    d = Dist(args.gpus)
    line = {"n_gpus": d.world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "vs_baseline": None, "data": "synthetic"}
    if args.workload.startswith("attn_bwd"):
        r = bench_attention_bwd(d, args.workload.replace("_bwd", ""), args.steps, args.warmup, peaks)
        line.update({"metric": "attention_bwd_tflops", "scaling": "weak", "dtype": "bf16",
                     "config": {"workload": r.pop("workload"), "l2": "inputs larger than L2"}})
        line.update(r)
    elif args.workload.startswith("attn"):
        # the long-context shape is ONE job split over the GPUs (strong scaling); the others run per GPU
        split = "strong" if args.workload == "attn_c3" else "weak"
        r = bench_attention(d, args.workload, args.steps, args.warmup, peaks, with_e2e=not args.no_e2e, split=split)
        line.update({"metric": "attention_fwd_tflops", "unit": "TFLOP/s", "dtype": "bf16"})
        line.update(r)
    elif args.workload == "lion_c4":
        r = bench_lion_c4(d, args.steps, args.warmup, peaks, with_e2e=not args.no_e2e)
        line.update({"metric": "lion_step_hbm_gbs", "scaling": "weak", "dtype": "f32",
                     "config": {"workload": r.pop("workload"), "l2": "5.7 GB per step, larger than L2"}})
        line.update(r)
    else:
        r = bench_lion_c5(d, args.steps, args.warmup, peaks)
        line.update({"metric": "lion_step_hbm_gbs", "dtype": "bf16",
                     "config": {"workload": r.pop("workload"), "l2": "67 GB per step, larger than L2"}})
        line.update(r)

    if not args.no_also:
        also = {}
        if args.workload != "attn_c2":
            a = bench_attention(d, "attn_c2", max(args.steps, 50), args.warmup, peaks, with_e2e=False, with_clocks=False)
            also["attn_c2"] = {k: a[k] for k in ("value", "ms_per_step", "roofline", "config")}
            also["attn_c2"]["unit"] = "TFLOP/s"
        if args.workload == "attn_c3" and d.world > 1:
            a = bench_attention(d, "attn_c3", max(3, args.steps // 2), args.warmup, peaks, with_e2e=False,
                                with_clocks=False, split="weak")
            also["attn_c3_weak"] = {k: a[k] for k in ("value", "ms_per_step", "scaling", "roofline", "config")}
            also["attn_c3_weak"]["unit"] = "TFLOP/s"
        if not args.workload.startswith("attn_bwd"):
            also["attn_bwd_c3"] = bench_attention_bwd(d, "attn_c3", max(3, args.steps // 4), 2, peaks)
            also["attn_bias_dropout_c3"] = bench_attention_variants(d, "attn_c3", max(3, args.steps // 4), 2, peaks)
            also["attn_sweep"] = bench_attention_sweep(d, max(10, args.steps // 2), 5, peaks)
        if args.workload != "lion_c4":
            also["lion_c4"] = bench_lion_c4(d, args.steps, args.warmup, peaks)
        if args.workload != "lion_c5":
            also["lion_c5"] = bench_lion_c5(d, max(3, args.steps // 4), 2, peaks)
        if d.world == 1:
            also["reference_points"] = bench_reference_points(d)
        line["also"] = also

    if d.rank == 0 and d.world == 1 and not args.no_cpu:
        if args.workload.startswith("attn_bwd"):
            pass
        elif args.workload.startswith("attn"):
            line["cpu_baseline"], _ = cpu_attention_sample(args.workload, 1, 3)
            if not args.no_also:
                line["also"]["lion_c4"]["cpu_baseline"] = cpu_lion_sample(3)
        else:
            line["cpu_baseline"] = cpu_lion_sample(3)
    d.close()
    if d.rank == 0:
        print(json.dumps(line), flush=True)
    # a failed ZeRO-1 self-check fails the run, after every rank has left the group in order
    text = json.dumps(line)
    if '"parity_check": "FAILED' in text:
        raise SystemExit("ZeRO-1 parity check failed: see parity_check in the line above")


if __name__ == "__main__":
    main()
