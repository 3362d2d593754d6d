#!/usr/bin/env python
"""Benchmark of the CRF-CTC decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode of one batch of synthetic scores: hac model, state_len 4, T = 1666,
N = 512 chunks per GPU, C = 1024, fp16 (the single-GPU configuration the headline metric is
quoted on).  With N GPUs every rank decodes its own 512 chunks (chunks are independent, so the
batch is sharded by chunk index with no data-path collective; weak scaling).

`value` is decoded chunks per second with the scores already resident in HBM, timed on the
device with the CUDA events the library records on the stream its kernels run on; `e2e` is the
same metric through openfish_decode_gpu with the scores starting in (page-locked) host memory
and the results ending in host memory.  `roofline` describes the kernel that takes the most
device time; `cpu_baseline` is the reference CPU decoder on this box's host cores on a bounded
sample.  One JSON line is printed by rank 0.

Outside the timed region the line also carries: `parity_spot_check` (every rank compares the
first chunks of its shard with the CPU oracle, so that every GPU's output gets checked, not only
the first one's), `config3_strong` (4096 chunks in all, split evenly over the ranks: strong
scaling) and, on one GPU, `other_models` (the 1024-state and the 64-state model) and
`blank_column_adaptor` (the entry point for scores that carry the blank column).
"""
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

STATE_LEN, T, N_PER_GPU = 4, 1666, 512
NS = 4 ** STATE_LEN
C = 4 * NS
SEED = 0x0F16
METRIC = "decoded chunks/sec (hac, T=1666)"
UNIT = "chunks/s"
WORKLOAD = ("hac CRF decode: state_len=4 (256 states), T=1666, N=%d chunks per GPU, C=1024 fp16 "
            "[T][N][C], 5*tanh(1.5z)+4 planted path, DECODER_INIT options" % N_PER_GPU)

CONFIG = {"workload": WORKLOAD,
          "l2": "inputs (1.75 GB scores + 0.87 GB bwd per GPU) exceed the 126 MB L2; no flush needed",
          "sharding": "by chunk index, one rank per GPU, no collective"}

# algorithmic bytes per chunk (fp16 scores read once per scan; bwd written then read; post,
# moves, sequence, qstring written)
B_KERNEL = {"bwd_scan": T * 4 * NS * 2 + (T + 1) * NS * 4,              # scores in, bwd out
            "fwd_scan": T * 4 * NS * 2 + 2 * (T + 1) * NS * 4,          # scores, bwd in; post out (forward scan + posterior)
            # what the search needs: <= 128 fp16 scores and <= 160 fp32 backward scores gathered per
            # timestep, one back-pointer byte per slot out (the rows it streams to find them are
            # traffic, not algorithmic bytes)
            "beam_search": T * (128 * 2 + 160 * 4) + 32 * (T + 1),
            "posterior_seq": 32 * (T + 1) + 9 * 4 * T + 3 * T}          # back-pointers, <= 9 posteriors per step in; results out


def chunk_bytes(state_len, t):
    """Algorithmic bytes of one chunk's decode: scores read once per scan; bwd written then read;
    post, moves, sequence, qstring written."""
    ns = 4 ** state_len
    return 2 * t * 4 * ns * 2 + 3 * (t + 1) * ns * 4 + 3 * t


B_CHUNK = chunk_bytes(STATE_LEN, T)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def ncu_traffic(kernel):
    """DRAM bytes per launch of `kernel` from the committed ncu summary, if there is one."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)).get(kernel)
        except Exception:
            return None
    return None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.sm_max = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
                 "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80)}
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = get(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def finish(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.sm_max,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def measure_rotary(of, dev, cpu_too=False):
    """openfish_rotary_emb_gpu on fp16 [32][1666][3][8][64] (Q and K heads in one call): device time
    by the library's CUDA events on the legacy default stream the kernel runs on, rotating over four tensors
    (655 MB) so that no call finds its input in the 126 MB L2."""
    import numpy as np
    import torch
    B, S, H, D = 32, 1666, 8, 64
    half = D // 2
    pos = np.arange(S)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    sin = torch.from_numpy(np.sin(pos).astype(np.float32)).to(dev)
    cos = torch.from_numpy(np.cos(pos).astype(np.float32)).to(dev)
    g = torch.Generator(device=dev).manual_seed(4)
    xs = [torch.randn((B, S, 3, H, D), generator=g, device=dev, dtype=torch.float32).half() for _ in range(4)]
    args = (B, S, 2 * H, D, half, S * 3 * H * D, 3 * H * D, D)
    for x in xs:
        of.rotary_emb_gpu(x, sin, cos, *args)
    reps, total, wall = 20, 0.0, 0.0
    for i in range(reps):
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        of.rotary_emb_gpu(xs[i % 4], sin, cos, *args)
        wall += time.perf_counter() - w0
        total += of.last_rotary_ms()  # the library's own events around the kernel
    ms = total / reps
    nbytes = 2 * B * S * 2 * H * D * 2 + 2 * S * half * 4
    peak, _ = measured_peak()
    out = {"shape": "fp16 [32][1666][3][8][64], nheads=16", "ms": ms, "algorithmic_bytes": nbytes,
            "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peak,
            "call_wall_ms": 1e3 * wall / reps, "calls": reps}
    if cpu_too:
        # the reference's CPU routine on the same values widened to float32 (it works on float32),
        # all host cores (it caps its threads at the batch size, src/nn_cpu.c:95)
        import oracle
        x32 = xs[0].float().cpu().numpy().reshape(-1)
        cores = os.cpu_count() or 1
        fn, kind = (oracle.ref_rotary, "reference") if oracle.have_ref() else (None, "port")
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            if fn:
                fn(x32, sin.cpu().numpy(), cos.cpu().numpy(), half, S * 3 * H * D, 3 * H * D, D, B, S, 2 * H, cores)
            else:
                oracle.rotary(x32, sin.cpu().numpy(), cos.cpu().numpy(), half, S * 3 * H * D, 3 * H * D, D, B, S, 2 * H)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        out["cpu_baseline"] = {"ms": 1e3 * best, "kind": kind, "cores": min(cores, B) if fn else 1}
    return out


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def cpu_decode_rate(scores32, threads, repeats=1):
    """chunks/s of the reference CPU decoder (the compiled reference when present, else the
    restatement) on a float32 [T][n][C] sample."""
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    fn = oracle.ref_decode if kind == "reference" else oracle.decode
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn(scores32, STATE_LEN, None, threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return scores32.shape[1] / best, kind, best


def host_sample(n_chunks, seed):
    import numpy as np
    from openfish_b200 import synth
    return synth.make_scores(T, n_chunks, STATE_LEN, seed).astype(np.float32)


def run_reference(args, rank, world):
    """The reference arm: the reference's own CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    n = min(N_PER_GPU, max(cores, 256))  # a bounded sample of the workload per step (about a second)
    sc = host_sample(n, SEED)
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_decode_rate(sc, cores)
    times, kind = [], "port"
    for _ in range(args.steps):
        rate, kind, dt = cpu_decode_rate(sc, cores)
        times.append(dt)
    total = sum(times)
    value = n * len(times) / total
    config = dict(CONFIG, workload=WORKLOAD + "; this arm decodes a %d-chunk sample of it per step (the CPU "
                  "decoder works chunk by chunk, so its chunks/s does not depend on the batch size)" % n)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 storage, f64 exp/log (the CPU decoder's arithmetic)", "data": "synthetic",
            "config": config, "sample_chunks_per_step": n,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": min(cores, n), "kind": kind,
                             "sample": "%d chunks of the workload per step, openfish_decode_cpu with %d threads" % (n, min(cores, n))},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def timed_decodes(of, scores, state_len, steps, warmup=3):
    """Median device time (the library's own CUDA events) of `steps` decodes of a resident batch,
    after `warmup` untimed ones; also the decoded bases of the batch."""
    import torch
    t, n, _ = scores.shape
    gb = of.gpubuf_init(t, n, state_len)
    res = [torch.empty((n, t), dtype=torch.uint8).pin_memory() for _ in range(3)]
    ms = []
    for k in range(warmup + steps):
        of.decode_into(scores, state_len, gb, *res)
        if k >= warmup:
            ms.append(gb.last_decode_ms())
    gb.free()
    med = {k: statistics.median(m[k] for m in ms) for k in ms[0]}
    return med, float(res[0].sum())


def other_model(of, dev, state_len, t, n, seed, peak):
    """One more model/shape with the same kernels, scores resident: ms per decode, chunks/s and the
    whole-decode roofline on that shape's own algorithmic bytes."""
    from openfish_b200 import synth
    scores = synth.make_scores_device(t, n, state_len, seed, dev)
    med, bases = timed_decodes(of, scores, state_len, steps=5)
    del scores
    gbs = chunk_bytes(state_len, t) * n / (med["total"] * 1e-3) / 1e9
    return {"state_len": state_len, "T": t, "N": n, "ms_per_decode": med["total"],
            "chunks_per_sec": n / (med["total"] * 1e-3), "bases_per_sec": bases / (med["total"] * 1e-3),
            "kernel_ms": {k: med[k] for k in ("bwd_scan", "fwd_scan", "beam_search", "posterior_seq", "d2h")},
            "roofline_whole_decode": {"achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                      "algorithmic_bytes_per_chunk": chunk_bytes(state_len, t)}}


def blank_column_adaptor(of, dev, peak):
    """The 5-wide entry point on the headline shape: device time of the kernel that strips the
    blank column (an HBM-bound streaming pass: 10*ns bytes in, 8*ns out per chunk and timestep)
    and of the whole call, scores resident."""
    import torch
    from openfish_b200 import synth
    wide = torch.empty((T, N_PER_GPU, 5 * NS), dtype=torch.float16, device=dev)
    t_block = 64
    for t0 in range(0, T, t_block):  # built in slices: the 4-wide scores with a stay column in front
        four = synth.make_scores_device(min(t_block, T - t0), N_PER_GPU, STATE_LEN, SEED + 1 + t0, dev)
        v = wide[t0:t0 + four.shape[0]].view(four.shape[0], N_PER_GPU, NS, 5)
        v[..., 1:] = four.view(four.shape[0], N_PER_GPU, NS, 4)
        v[..., 0] = 2.0
        del four
    gb = of.gpubuf_init(T, N_PER_GPU, STATE_LEN)
    res = [torch.empty((N_PER_GPU, T), dtype=torch.uint8).pin_memory() for _ in range(3)]
    strip, total = [], []
    for r in range(8):
        of.decode_5wide_into(wide, STATE_LEN, gb, *res, clamp=5.0)
        if r >= 3:
            ms = gb.last_decode_ms()
            strip.append(ms["strip_blank"])
            total.append(ms["strip_blank"] + ms["total"])
    gb.free()
    del wide
    torch.cuda.empty_cache()
    nbytes = 18.0 * NS * T * N_PER_GPU
    ms = statistics.median(strip)
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"shape": "fp16 [%d][%d][%d] -> [%d][%d][%d]" % (T, N_PER_GPU, 5 * NS, T, N_PER_GPU, 4 * NS),
            "strip_ms": ms, "strip_plus_decode_ms": statistics.median(total),
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "algorithmic_bytes_per_launch": nbytes},
            "timing": "library CUDA events, median of 5 calls after 3 warm-ups; 3.9 GB per launch, no L2 reuse"}


def spot_check(of, scores, results, state_len, n_check):
    """The first n_check chunks of this rank's batch through the CPU oracle (the checker, outside
    every timed region): how many have moves and sequence identical to what the GPU returned."""
    import numpy as np
    import oracle
    sub = scores[:, :n_check, :].float().cpu().numpy()
    ref = oracle.decode(np.ascontiguousarray(sub), state_len, None, min(n_check, os.cpu_count() or 1))
    same = 0
    for c in range(n_check):
        same += int(np.array_equal(results[0][c].numpy(), ref["moves"][c])
                    and np.array_equal(results[1][c].numpy(), ref["sequence"][c]))
    return same


def reference_cuda():
    """The reference's own CUDA kernels (generic code, compiled for sm_100a by baseline/Makefile)
    timed on this GPU by a child process; None of this library's code runs there, and nothing of
    the reference's runs in this process."""
    import subprocess
    script = os.path.join(ROOT, "baseline", "time_reference_cuda.py")
    try:
        r = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=300)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's CUDA path did not finish within 300 s"}
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    if r.returncode != 0 or not lines:
        tail = (r.stderr or "").strip().splitlines()[-1:] or [""]
        return {"unavailable": "the reference's CUDA path ended with code %d: %s" % (r.returncode, tail[0][:200])}
    return json.loads(lines[-1])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true")
    ap.add_argument("--profile", type=int, metavar="CHUNKS", default=0,
                    help="for captures under a profiler: decode CHUNKS chunks --warmup + --steps times, nothing else")
    ap.add_argument("--profile-model", type=int, default=STATE_LEN, help="state_len of the --profile decode (3, 4 or 5)")
    ap.add_argument("--profile-timesteps", type=int, default=T, help="T of the --profile decode")
    ap.add_argument("--profile-rotary", action="store_true",
                    help="for captures under a profiler: the rotary measurement alone (24 calls on the encoder's QKV shape)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import openfish_b200 as of
    from openfish_b200 import sharding, synth

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.profile_rotary:
        print(json.dumps({"rotary": measure_rotary(of, dev)}), flush=True)
        return
    if args.profile:
        # the same decode call on a smaller batch, so that a profiler's capture stays small
        sl = args.profile_model
        sc = synth.make_scores_device(args.profile_timesteps, args.profile, sl, SEED, dev)
        med, _ = timed_decodes(of, sc, sl, steps=args.steps, warmup=args.warmup)
        print(json.dumps({"profile_chunks": args.profile, "state_len": sl, "T": args.profile_timesteps, "ms": med}),
              flush=True)
        return

    # this rank's shard: chunks [rank*512, (rank+1)*512) of the job, generated in its own HBM
    lo, hi = sharding.shard_range(N_PER_GPU * world, rank, world)
    n_local = hi - lo
    scores = synth.make_scores_device(T, n_local, STATE_LEN, SEED, dev, first_chunk=lo)
    gb = of.gpubuf_init(T, n_local, STATE_LEN)
    res = [torch.empty((n_local, T), dtype=torch.uint8).pin_memory() for _ in range(3)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput (value) -------------------------------------------
    for _ in range(args.warmup):
        of.decode_into(scores, STATE_LEN, gb, *res)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    sampler.start()
    ms = {}
    w0 = time.perf_counter()
    for _ in range(args.steps):
        of.decode_into(scores, STATE_LEN, gb, *res)
        for k, v in gb.last_decode_ms().items():
            ms[k] = ms.get(k, 0.0) + v
    barrier()
    wall = time.perf_counter() - w0
    bases_local = float(res[0].sum())
    dev_s = sharding.max_over_ranks(ms["total"] * 1e-3, dev if world > 1 else None)
    wall_s = sharding.max_over_ranks(wall, dev if world > 1 else None)
    total_chunks = N_PER_GPU * world
    value = total_chunks * args.steps / dev_s
    bases = sharding.sum_over_ranks(bases_local, dev if world > 1 else None)

    # ---- end to end through the reference-facing call, host buffers -----------------------
    # Two host threads, each with its own device score buffer and gpubuf, take the steps in turn:
    # while one is inside openfish_decode_gpu the other copies its next batch in on a stream of
    # its own (the reference's threading model, src/main.c:23,207: a gpubuf and a score buffer
    # per host thread).  Every step's host-to-device copy and result read-back is in the region.
    h_scores = torch.empty(scores.shape, dtype=torch.float16).pin_memory()
    h_scores.copy_(scores)
    e2e_steps = max(4, min(args.steps, 10))
    lanes = 2
    d_ins = [torch.empty_like(scores) for _ in range(lanes)]
    gbs = [gb] + [of.gpubuf_init(T, n_local, STATE_LEN) for _ in range(lanes - 1)]
    errors = []

    def e2e_lane(k, count):
        try:
            torch.cuda.set_device(local_rank)  # the library decodes on the calling thread's device
            st = torch.cuda.Stream(device=dev)
            for _ in range(count):
                with torch.cuda.stream(st):
                    d_ins[k].copy_(h_scores, non_blocking=True)
                st.synchronize()
                out = of.decode_gpu(d_ins[k], STATE_LEN, gpubuf=gbs[k])  # results malloc'ed on the host
                _ = int(out["moves"][0, 0])
        except Exception as exc:  # surfaced after the join
            errors.append(exc)

    def e2e_run(total_steps):
        per = [total_steps // lanes + (1 if k < total_steps % lanes else 0) for k in range(lanes)]
        th = [threading.Thread(target=e2e_lane, args=(k, per[k])) for k in range(lanes)]
        barrier()
        e0 = time.perf_counter()
        for t in th:
            t.start()
        for t in th:
            t.join()
        barrier()
        if errors:
            raise errors[0]
        return time.perf_counter() - e0

    e2e_run(lanes)  # warm-up: one step per lane
    e2e_s = sharding.max_over_ranks(e2e_run(e2e_steps), dev if world > 1 else None)

    # ---- two batches in flight on the device (scores resident): what a caller gets that submits
    # the next decode before waiting for the previous one (openfish_b200_decode_submit/_wait)
    res2 = [torch.empty((n_local, T), dtype=torch.uint8).pin_memory() for _ in range(3)]
    bufs = [(gbs[0], res), (gbs[1], res2)]

    def overlapped(steps):
        barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            g, r = bufs[i % 2]
            if i >= 2:
                of.decode_wait(g)
            of.decode_into(scores, STATE_LEN, g, *r, wait=False)
        for g, _ in bufs:
            of.decode_wait(g)
        barrier()
        return time.perf_counter() - t0

    overlapped(4)
    ov_steps = max(4, args.steps)
    ov_s = sharding.max_over_ranks(overlapped(ov_steps), dev if world > 1 else None)
    for g in gbs[1:]:
        g.free()
    clocks = sampler.finish()
    e2e_value = total_chunks * e2e_steps / e2e_s

    # ---- wall time of openfish_decode_gpu itself, scores resident (what the reference's driver
    # times, src/main.c:271-303), and the rotary helper on the encoder's packed QKV shape ------
    api_wall = []
    for _ in range(10):
        torch.cuda.synchronize()
        api_wall.append(of.decode_gpu_wall_ms(scores, STATE_LEN, gb))
    rotary = measure_rotary(of, dev, cpu_too=(world == 1 and not args.no_cpu_baseline)) if rank == 0 else None

    # ---- outside the timed regions ---------------------------------------------------------
    # every rank checks the head of its own shard against the oracle: the last timed decode's
    # results are still in `res`
    of.decode_into(scores, STATE_LEN, gb, *res)
    n_check = min(8, n_local)
    same = spot_check(of, scores, res, STATE_LEN, n_check)
    checked_total = sharding.sum_over_ranks(float(n_check), dev if world > 1 else None)
    same_total = sharding.sum_over_ranks(float(same), dev if world > 1 else None)
    gb.free()
    h2d_bytes = int(scores.numel() * 2)
    del scores, d_ins, h_scores
    torch.cuda.empty_cache()

    # BASELINE configuration 3 as written: 4096 chunks in all, split evenly by chunk index (strong
    # scaling; on one GPU all 4096, 14 GB of scores)
    n_strong = 4096
    s_lo, s_hi = sharding.shard_range(n_strong, rank, world)
    sc3 = synth.make_scores_device(T, s_hi - s_lo, STATE_LEN, SEED, dev, first_chunk=s_lo)
    barrier()
    med3, bases3 = timed_decodes(of, sc3, STATE_LEN, steps=3, warmup=3)
    del sc3
    torch.cuda.empty_cache()
    strong_ms = sharding.max_over_ranks(med3["total"], dev if world > 1 else None)
    strong_bases = sharding.sum_over_ranks(bases3, dev if world > 1 else None)
    peak_gbs, _ = measured_peak()
    config3 = {"chunks_total": n_strong, "chunks_per_gpu": s_hi - s_lo, "ms_per_decode": strong_ms,
               "chunks_per_sec": n_strong / (strong_ms * 1e-3), "bases_per_sec": strong_bases / (strong_ms * 1e-3),
               "per_gpu_hbm_gbs": B_CHUNK * (s_hi - s_lo) / (strong_ms * 1e-3) / 1e9,
               "scaling": "strong", "timing": "median of 3 decodes after 3 warm-ups, library CUDA events, max over ranks"}
    others = adaptor = None
    if world == 1:
        adaptor = blank_column_adaptor(of, dev, peak_gbs)
        others = [other_model(of, dev, 5, 1666, 256, 0x0F17, peak_gbs),
                  other_model(of, dev, 3, 1000, 16, 0x0F15, peak_gbs),
                  other_model(of, dev, 3, 1666, 1024, 0x0F15, peak_gbs)]

    if rank == 0:
        peak, peak_src = measured_peak()
        per = {k: v / args.steps for k, v in ms.items()}
        # The dominant kernel is the scan kernel (one template, launched once per direction:
        # together the largest share of device time); its figure is taken over both launches.
        groups = {"scan": ("bwd_scan", "fwd_scan"), "beam_search": ("beam_search",),
                  "posterior_seq": ("posterior_seq",)}
        dom = max(groups, key=lambda g: sum(per[k] for k in groups[g]))
        launches = groups[dom]
        dom_bytes = sum(B_KERNEL[k] for k in launches) * n_local / len(launches)
        dom_ms = sum(per[k] for k in launches) / len(launches)
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        whole = B_CHUNK * n_local / (per["total"] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dev_s / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 storage, f64 inside the log-sum-exp, fp16 scores", "data": "synthetic",
            "config": CONFIG, "chunks_total": total_chunks,
            "timing": "CUDA events recorded by the library on its own stream, summed over steps, max over ranks",
            "bases_per_sec": bases * args.steps / dev_s,
            "wall_ms_per_step": 1e3 * wall_s / args.steps,
            "kernel_ms": {k: per[k] for k in ("bwd_scan", "fwd_scan", "beam_search", "posterior_seq", "d2h")},
            "kernel_overlap": "fwd_scan (forward scan + posterior) runs on a second stream beside beam_search; the others are sequential",
            "roofline": {"bound": "hbm", "kernel": dom, "launches_per_decode": len(launches),
                         "avg_launch_ms": dom_ms, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": ncu_traffic(dom), "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": dom_bytes},
            "roofline_whole_decode": {"achieved": whole, "peak": peak, "unit": "GB/s", "frac": whole / peak,
                                      "algorithmic_bytes_per_chunk": B_CHUNK,
                                      "frac_of_nominal_8000_gbs": whole / 8000.0},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": int(3 * n_local * T), "steps": e2e_steps,
                    "call": "openfish_decode_gpu after a page-locked host-to-device copy of the scores; "
                            "two host threads alternate so that one's copy overlaps the other's decode"},
            "gpu_launches": of.lib().openfish_b200_kernels_per_decode() * args.steps * world,
            "decode_gpu_wall_ms": {"best": min(api_wall), "median": statistics.median(api_wall), "calls": 10,
                                   "note": "openfish_decode_gpu, scores resident, results malloc'ed on the host"},
            "two_in_flight": {"value": total_chunks * ov_steps / ov_s, "unit": UNIT, "ms_per_step": 1e3 * ov_s / ov_steps,
                              "steps": ov_steps, "timing": "wall clock between device synchronisations",
                              "note": "two gpubufs, the next decode submitted before the previous one is waited for"},
            "rotary": rotary,
            "clocks": clocks,
            "parity_spot_check": {"chunks_checked": int(checked_total), "identical": int(same_total),
                                  "what": "moves and sequence of the first %d chunks of every rank's shard against the CPU oracle" % n_check},
            "config3_strong": config3,
            "other_models": others,
            "blank_column_adaptor": adaptor,
        }
        if world == 1 and not args.no_reference_cuda:
            rc = reference_cuda()
            if "decode_hac_N512" in rc:
                rc["decode_hac_N512"]["this_library_ms"] = min(api_wall)
                rc["decode_hac_N512"]["speedup_wall"] = rc["decode_hac_N512"]["wall_ms"] / min(api_wall)
            if rc.get("rotary") and rotary:
                rc["rotary"]["this_library_ms"] = rotary["ms"]
                rc["rotary"]["speedup"] = rc["rotary"]["ms"] / rotary["ms"]
            line["reference_cuda"] = rc
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            n_s = min(N_PER_GPU, max(cores, 256))
            sc32 = synth.make_scores_device(T, n_s, STATE_LEN, SEED, dev).float().cpu().numpy()
            rate, kind, dt = cpu_decode_rate(np.ascontiguousarray(sc32), cores)
            line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": min(cores, n_s), "kind": kind,
                                    "sample": "first %d chunks of the same batch, one openfish_decode_cpu call, %.2f s" % (n_s, dt)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
