#!/usr/bin/env python
"""Benchmark of the fused BERT encoder path.

Workload (one "step"): the 12-layer BERT-base encoder over a batch of 64 sequences of 128 tokens
with random valid lengths in [32, 128] (seeded synthetic weights and activations), sharded by
sequence across the GPUs of one node; with more than one GPU the step ends with one NCCL
all-gather of the outputs.  Metric: sequences per second over all GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  `value` is timed with inputs resident in HBM; `e2e` is the same step through
the host-buffer entry point (pinned host input -> device -> encoder -> host output).  The batch-1
latencies of one layer and of the 12-layer stack are reported under `latency_us`.
`stages` carries the per-stage time of one layer at batch 1 and at batch 64 from the kernel's own stage clocks.
`--impl reference` times the CPU restatement of the reference model (oracle/) on the host cores: the whole batch
of 64 sequences per step, for exactly the steps and warm-ups asked for.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, SEQ, HEADS, HEAD_DIM, FFN, LAYERS = 64, 128, 12, 64, 3072, 12
HIDDEN = HEADS * HEAD_DIM
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the timed kernel at every shard size of this benchmark,
# {sequences per GPU: bytes}, each from a one-pass capture of the 12-layer launch of that many sequences
#   ncu --metrics gpu__time_duration.sum,dram__bytes_read.sum,dram__bytes_write.sum --clock-control none \
#       -k regex:souffle_megakernel -s 4 -c 1 --csv python -m souffle_models_b200.profile_cases bert_base_b<n>
# (the library as of the commit that introduced this table; tilings chosen by the cycle model, not timed)
DRAM_BYTES_PER_LAUNCH = {64: 357_393_152 + 494_891_264, 32: 179_636_224 + 19_077_632, 16: 173_738_240 + 4_755_456,
                         8: 171_836_160 + 4_379_392}
METRIC = "bert_base_12layer_seq128_batch64_sequences_per_second"
WORKLOAD = "BERT-base 12-layer encoder, batch 64 (sharded by sequence), seq 128, lengths U[32,128]"
SEED = 1239


def layer_flops(batch: int, seq: int = SEQ) -> int:
    """Algorithmic FLOPs of one encoder layer (padded-dense count): QKV, QK^T and PV, proj, FC1, FC2."""
    m = batch * seq
    return 2 * m * HIDDEN * 3 * HIDDEN + 2 * batch * HEADS * seq * seq * HEAD_DIM * 2 + 2 * m * HIDDEN * HIDDEN \
        + 2 * m * HIDDEN * FFN * 2


def layer_weight_bytes() -> int:
    return (4 * HIDDEN * HIDDEN + 2 * HIDDEN * FFN) * 2 + (3 * HIDDEN + HIDDEN + FFN + HIDDEN + 4 * HIDDEN) * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(tflops=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"], hbm=d["hbm_gbs"], src="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._stop_ev = index, [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        while not self._stop_ev.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def stop(self):
        self._stop_ev.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_workload(n_seq: int):
    from oracle import souffle_oracle as so
    cfg = so.BertConfig(n_seq, SEQ, HEADS, HEAD_DIM, FFN, "std")
    layers = so.make_bert_weights(cfg, SEED, LAYERS)
    full = so.BertConfig(BATCH, SEQ, HEADS, HEAD_DIM, FFN, "std")
    x, lens = so.make_bert_input(full, SEED, ragged=True)
    return so, cfg, layers, x, lens


def cpu_sample(n_seq: int, steps: int, warmup: int):
    """Times the CPU restatement of the reference model on `n_seq` sequences of the workload."""
    so, cfg, layers, x, lens = make_workload(n_seq)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    xs, ls = x[:n_seq], lens[:n_seq]
    with torch.no_grad():
        for _ in range(warmup):
            so.bert_stack(cfg, xs, layers, ls)
        t0 = time.perf_counter()
        for _ in range(steps):
            so.bert_stack(cfg, xs, layers, ls)
        dt = (time.perf_counter() - t0) / steps
    return n_seq / dt, dt, cores


def run_reference(args, rank: int, world: int):
    """The reference arm: the CPU restatement of the reference model on all host threads, the whole batch of 64
    sequences per step, exactly `--warmup` untimed and `--steps` timed passes."""
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    value, dt, cores = cpu_sample(BATCH, steps, warmup)
    sample = f"all {BATCH} sequences per step (12 layers, fp32 torch-CPU restatement of python/models/bert/bert_torch.py)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "sequences/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1000.0,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "sequences/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def timed(fn, steps: int, barrier, drain=None):
    """K calls of fn between two CUDA events on the current stream; `drain` (optional) makes the current stream
    wait for work fn left on other streams, so that the closing event covers it."""
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if drain is not None:
        drain()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps          # ms per step


def latency_us(bert, so, n_layers: int, iters: int = 200) -> float:
    """Batch-1, seq-128 latency per call in microseconds: back-to-back launches, weights hot in L2 for
    one layer (14 MB) and streamed from HBM for twelve (170 MB)."""
    cfg = so.BertConfig(1, SEQ, HEADS, HEAD_DIM, FFN, "std")
    layers = [{k: v.cuda() for k, v in w.items()} for w in so.make_bert_weights(cfg, SEED + 1, n_layers)]
    enc = bert.BertEncoder(1, SEQ, HEADS, HEAD_DIM, FFN, layers)
    x = so.make_bert_input(cfg, SEED + 1)[0].cuda()
    y = torch.empty_like(x)
    for _ in range(20):
        enc.forward(x, None, y)
    ms = timed(lambda: enc.forward(x, None, y), iters, lambda: None)
    enc.status()
    enc.close()
    return ms * 1000.0


def latency_cold_us(bert, so, iters: int = 30) -> float:
    """Batch-1, seq-128, one layer with its weights cold: a 256 MB buffer is rewritten before every call (twice the
    L2), one call between each pair of events, median over `iters` in microseconds.  This is the case the HBM floor
    of a single layer applies to."""
    cfg = so.BertConfig(1, SEQ, HEADS, HEAD_DIM, FFN, "std")
    layers = [{k: v.cuda() for k, v in w.items()} for w in so.make_bert_weights(cfg, SEED + 1, 1)]
    enc = bert.BertEncoder(1, SEQ, HEADS, HEAD_DIM, FFN, layers)
    x = so.make_bert_input(cfg, SEED + 1)[0].cuda()
    y = torch.empty_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(5):
        enc.forward(x, None, y)
    pairs = []
    for i in range(iters):
        flush.fill_(i & 0xFF)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        enc.forward(x, None, y)
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    enc.status()
    enc.close()
    ts = sorted(a.elapsed_time(b) for a, b in pairs)
    return ts[len(ts) // 2] * 1000.0


_RESULT_FD = None


def emit(line: str) -> None:
    """The one result line goes to the process's original stdout."""
    if _RESULT_FD is None:
        print(line, flush=True)
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, (line + "\n").encode())


STAGE_NAMES = ("qkv", "attention", "proj", "ln1", "fc1", "fc2", "ln2")


def stage_profile(bert, so, batch: int, mhz: float):
    """Per-stage time of ONE encoder layer at `batch` sequences from the kernel's own stage clocks (desc.profile):
    work (stage start -> the CTA reaches the grid barrier; median over the CTAs and the slowest CTA) and barrier wait
    (median), in SM cycles, and the median CTA's work + wait in microseconds at `mhz`.  `kernel_us` is the wall clock
    from the first CTA's entry to the last CTA's exit."""
    cfg = so.BertConfig(batch, SEQ, HEADS, HEAD_DIM, FFN, "std")
    layers = [{k: v.cuda() for k, v in w.items()} for w in so.make_bert_weights(cfg, SEED + 2, 1)]
    enc = bert.BertEncoder(batch, SEQ, HEADS, HEAD_DIM, FFN, layers, tuning={"profile": 1, "autotune": 1})
    x, lens = so.make_bert_input(cfg, SEED + 2, ragged=batch > 1)
    xs, ls = x.cuda(), (lens.cuda() if lens is not None else None)
    y = torch.empty_like(xs)
    for _ in range(5):
        enc.forward(xs, ls, y)
    enc.status()
    pr = enc.read_profile().double()
    out = {}
    for si, name in enumerate(STAGE_NAMES):
        w = pr[si, :, 1] - pr[si, :, 0]
        work = w.median().item()
        bar = (pr[si, :, 2] - pr[si, :, 1]).median().item() if si + 1 < len(STAGE_NAMES) else 0.0
        out[name] = {"work_cycles": work, "work_cycles_max": w.max().item(), "barrier_cycles": bar, "us": (work + bar) / mhz}
    k = pr[-1]
    out["kernel_us"] = (k[:, 4].max() - k[:, 3].min()).item() / 1000.0      # first CTA in -> last CTA out, wall clock
    enc.close()
    return out


def run_ours(args, rank: int, world: int, local_rank: int):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    import torch.distributed as dist
    from souffle_models_b200 import bert, sharding
    per = BATCH // world
    so, cfg, layers, x, lens = make_workload(per)
    xs, ls = sharding.shard_batch(x, lens, rank, world)
    dev_layers = [{k: v.cuda() for k, v in w.items()} for w in layers]
    # every rank runs the same tilings (rank 0 times them, the others take its choice): identical work per rank, and
    # outputs that do not depend on which rank computed a sequence
    enc = sharding.encoder_with_common_tiling(
        lambda tuning: bert.BertEncoder(per, SEQ, HEADS, HEAD_DIM, FFN, dev_layers, tuning=tuning), rank, world)
    x_d, l_d = xs.cuda(), ls.cuda()
    y_d = torch.empty_like(x_d)
    full = torch.empty(BATCH, SEQ, HIDDEN, dtype=torch.float16, device="cuda") if world > 1 else None

    def barrier():
        if world > 1:
            dist.barrier()

    def step():
        enc.forward(x_d, l_d, y_d)
        if world > 1:
            sharding.gather_outputs(y_d, full)

    # end to end: pinned host shard in, this rank's slice of the (gathered) result back to pinned host memory, every
    # step; one GPU goes through the library's own host-buffer entry point, several through the package's pipeline
    x_h, y_h, l_h = xs.pin_memory(), torch.empty_like(xs).pin_memory(), ls.pin_memory()
    pipe = sharding.ShardedHostPipeline(enc.forward, x_d, l_d, rank, world) if world > 1 else None

    def step_e2e():
        if world == 1:
            enc.forward_host(x_h, l_h, y_h, wait=False)
        else:
            pipe.step(x_h, l_h, y_h)

    def drain_e2e():
        if pipe is not None:
            pipe.drain()

    for _ in range(max(3, args.warmup)):
        step()
    enc.status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step, args.steps, barrier)
    clocks = sampler.stop()
    enc.status()
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps, barrier, drain_e2e)
    enc.status()
    info = enc.info()
    # outside the timed region: what every rank computed and gathered equals, bit for bit, what ONE GPU computes for
    # the same sequences with the same plan (rank 0 runs every shard through its own encoder)
    gathered_ok = None
    if world > 1:
        step()
        torch.cuda.synchronize()
        if rank == 0:
            gathered_ok = True
            for r in range(world):
                xr, lr = sharding.shard_batch(x, lens, r, world)
                yr = enc.forward(xr.cuda(), lr.cuda())
                enc.status()
                gathered_ok = gathered_ok and bool(torch.equal(yr.reshape(per, SEQ, HIDDEN), full[r * per:(r + 1) * per]))
        t = torch.tensor([ms, ms_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = t[0].item(), t[1].item()
    if rank != 0:
        return
    peaks = measured_peaks()
    flops_step_gpu = layer_flops(per) * LAYERS
    achieved = flops_step_gpu / (ms * 1e-3) / 1e12
    lat, stages, cpu = {}, {}, None
    if world == 1:
        lat = {"bert_layer_b1_s128": latency_us(bert, so, 1), "bert_12layer_b1_s128": latency_us(bert, so, 12, 50)}
        hbm_floor_us = (layer_weight_bytes() + 2 * SEQ * HIDDEN * 2) / (peaks["hbm"] * 1e9) * 1e6
        lat["bert_layer_b1_s128_cold_l2"] = latency_cold_us(bert, so)
        lat["hbm_floor_layer_us"] = hbm_floor_us
        lat["hbm_frac_layer_cold_l2"] = hbm_floor_us / lat["bert_layer_b1_s128_cold_l2"]
        lat["hbm_frac_12layer"] = 12 * hbm_floor_us / lat["bert_12layer_b1_s128"]
        mhz = float(clocks.get("sm_max_mhz") or 1965.0)         # short launches run at the maximum clock
        stages = {"clock_mhz": mhz, "layer_b1_s128": stage_profile(bert, so, 1, mhz),
                  "layer_b64_s128": stage_profile(bert, so, BATCH, mhz)}
        n_seq = BATCH
        v, dt, cores = cpu_sample(n_seq, 3, 1)
        cpu = {"value": v, "unit": "sequences/s", "cores": cores, "kind": "port",
               "sample": f"{n_seq} of the {BATCH} sequences, 12 layers, fp32 torch-CPU oracle, {dt:.2f} s per pass"}
    out = {
        "metric": METRIC, "value": BATCH / (ms * 1e-3), "unit": "sequences/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "sequences_per_gpu": per, "parallelism": f"replicas x{world}, output all-gather" if world > 1 else "single GPU",
                   "l2": "no flush: 170 MB of weights per step exceed the 126 MB L2", "grid": info["grid"],
                   "stages_per_launch": info["stages"],
                   "tiles": "timed at plan creation (desc.autotune): " + ", ".join(
                       "%dx%d/%d" % (t["bm"], t["bn"], t["splitk"]) for t in (enc.stage_info(i) for i in (0, 2, 4, 5))),
                   "e2e": ("souffle_bert_forward_host_async: pinned host in/out per step; steps pipelined over copy-in, compute and copy-out streams"
                           if world == 1 else "sharding.ShardedHostPipeline: pinned host shard in, all-gather on the device, every rank reads its slice of the gathered result back; steps pipelined over three streams")},
        "e2e": {"value": BATCH / (ms_e2e * 1e-3), "unit": "sequences/s",
                "h2d_bytes_per_step": int((xs.numel() * 2 + ls.numel() * 4) * world),      # whole job: all ranks' shards
                "d2h_bytes_per_step": int(BATCH * SEQ * HIDDEN * 2)},
        "gpu_launches": args.steps * info["launches"],
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tflops"], "frac_of_sustained_peak": achieved / peaks["tflops_sustained"],
                     "peak_source": peaks["src"] + " (cuBLAS bf16 burst)",
                     "traffic": DRAM_BYTES_PER_LAUNCH.get(per),
                     "kernel": "souffle_megakernel", "flops_per_launch": flops_step_gpu},
        "clocks": clocks,
        "latency_us": lat,
    }
    if stages:
        out["stages"] = stages
    if gathered_ok is not None:
        out["gathered_equals_single_gpu"] = gathered_ok
    if cpu:
        out["cpu_baseline"] = cpu
    emit(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        # libraries print banners (the NCCL version) on the C-level stdout: send everything but the result line to stderr
        global _RESULT_FD
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
