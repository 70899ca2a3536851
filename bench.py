#!/usr/bin/env python
"""Benchmark of the fused GEMM + epilogue path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload k2] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input: one fused launch (the
`pipeline` workload: its four launches).  Default workload: k2 = GEMM + RMSNorm row-scale + SwiGLU
at the Llama-3-8B FFN gate/up shape (M=4096 tokens, K=4096, N=28672 interleaved gate/up columns,
output [4096,14336] bf16).  With N GPUs the weight columns are sharded N-ways (activations and
per-row scales replicated, nothing exchanged inside a stage), so total work is fixed: strong
scaling.  Prints ONE JSON line on rank 0.

  value     whole-job TFLOP/s (2*M*N*K per GEMM), inputs resident in HBM, CUDA-event timed,
            max over ranks
  e2e       the same metric through the C ABI with HOST buffers: every step copies the step's
            activations + row scales host->device from pinned memory and the output device->host
  roofline  tensor-core bound: achieved 2MNK / average launch time against the measured bf16 peak
  cpu_baseline / --impl reference
            the CPU oracle (a port of the reference's formulas; the reference has no CPU or CUDA
            implementation of its own) timed on the host cores on a bounded row-sample
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused GEMM+epilogue TFLOP/s"

# name -> list of stages: (preset, M, N, K, dtype[, "chain"]); a "chain" stage contracts over the
# previous stage's output (all-gathered across ranks when the columns are sharded)
WORKLOADS = {
    "k1": [("k1", 512, 4096, 4096, "bf16")],
    "k2": [("k2", 4096, 28672, 4096, "bf16")],
    "k4v2_q": [("k4v2", 4096, 4096, 4096, "bf16")],
    "k4v2_kv": [("k4v2", 4096, 1024, 4096, "bf16")],
    "w8a8": [("w8a8", 8192, 8192, 28672, "s8")],
    # Llama-3-70B decoder-layer GEMM chain, M = 8192 tokens
    "pipeline": [("k4v2", 8192, 10240, 8192, "bf16"), ("k0a", 8192, 8192, 8192, "bf16"),
                 ("k2", 8192, 57344, 8192, "bf16"), ("k0a", 8192, 8192, 28672, "bf16", "chain")],
}
DESCR = {
    "k1": "k1 GEMM+RMSNorm row-scale M=512 N=4096 K=4096 bf16",
    "k2": "k2 GEMM+RMSNorm+SwiGLU Llama-3-8B FFN gate/up M=4096 K=4096 N=28672 (interleaved) -> [4096,14336] bf16",
    "k4v2_q": "k4v2 GEMM+RMSNorm+RoPE Llama-3-8B Q-proj M=4096 K=4096 N=4096, table [4096,128] theta=5e5",
    "k4v2_kv": "k4v2 GEMM+RMSNorm+RoPE Llama-3-8B K-proj M=4096 K=4096 N=1024, table [4096,128] theta=5e5",
    "w8a8": "w8a8_dequant_biased Llama-3-70B FFN down M=8192 K=28672 N=8192 int8 -> bf16, bf16 bias",
    "pipeline": "Llama-3-70B layer GEMM chain M=8192: QKV k4v2 (K=8192,N=10240), O k0a (8192,8192), "
                "gate/up k2 (K=8192,N=57344), down k0a (K=28672,N=8192)",
}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the workload's kernel, from the
# ncu captures summarised under profiles/ (full-size workloads, one GPU).
NCU_DRAM_BYTES_PER_LAUNCH = {
    "k2": 507_871_488 + 108_579_584,       # profiles/gemm_evt_kernel_bf16_256x256_cta2_k128__k2_*.md
    "w8a8": 1_990_824_000 + 129_954_816,   # profiles/gemm_evt_kernel_s8_256x256_cta2_k256__w8a8_*.md
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16": d["bf16_tflops"], "bf16_sustained": d.get("bf16_tflops_sustained"),
                "hbm": d["hbm_gbs"], "src": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "src": "fallback"}


# ------------------------------------------------------------------------------ clocks sampler
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons of one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid = uuid
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", self.uuid], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0=None, t1=None, load_window=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = []
        for ts, l in self.lines:
            if t0 is not None and not (t0 - 0.05 <= ts <= t1 + 0.1):
                continue
            f = [x.strip() for x in l.split(",")]
            if len(f) >= 6 and f[0].isdigit():
                rows.append(f)
        if not rows:
            rows = [[x.strip() for x in l.split(",")] for _, l in self.lines
                    if l and l.split(",")[0].strip().isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        # the SM clock under load: samples of the window in which the timed step ran continuously
        load = []
        if load_window is not None:
            for ts, l in self.lines:
                f = [x.strip() for x in l.split(",")]
                if load_window[0] <= ts <= load_window[1] and len(f) >= 6 and f[0].isdigit():
                    load.append(int(f[0]))
        sm = sorted(load) if load else sorted(int(r[0]) for r in rows)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons,
                "samples": len(rows), "load_samples": len(load),
                "how": "sm_mhz = median over the untimed repeat of the timed step that follows it; "
                       "reasons over the whole run"}


# ------------------------------------------------------------------------------ synthetic inputs
def gen_stage_host(stage, rank, world, seed):
    """Seeded host tensors of one stage for this rank's column shard (pinned where copied per step)."""
    import torch
    preset, M, N, K, dt = stage[:5]
    chain = len(stage) > 5 and stage[5] == "chain"
    assert N % world == 0
    Ns = N // world
    g = torch.Generator().manual_seed(seed)
    gw = torch.Generator().manual_seed(seed * 7919 + 13 * rank + 1)   # per-shard weight stream
    h = {}
    if dt == "bf16":
        if chain:                      # activations come from the previous stage, on the device
            h["X"], h["R"] = None, None
        else:
            X = torch.randn(M, K, generator=g, dtype=torch.float32)
            h["R"] = torch.rsqrt((X * X).mean(dim=1) + 1e-6).contiguous()    # fp32 on the host
            h["X"] = X.to(torch.bfloat16)
        W = torch.empty(K, Ns, dtype=torch.bfloat16)
        for k0 in range(0, K, 4096):                                      # bounded temporaries
            k1 = min(K, k0 + 4096)
            W[k0:k1] = (torch.randn(k1 - k0, Ns, generator=gw) * K ** -0.5).to(torch.bfloat16)
        h["W"] = W
    else:
        X = torch.randn(M, K, generator=g, dtype=torch.float32).to(torch.bfloat16).float()
        st = X.abs().amax(dim=1) / 127.0 + 1e-8                          # per-token absmax
        h["X"] = torch.clamp(torch.round(X / st[:, None]), -128, 127).to(torch.int8)
        h["R"] = st.contiguous()
        W = torch.empty(K, Ns, dtype=torch.int8)
        sc = torch.zeros(Ns)
        Wf = torch.empty(K, Ns, dtype=torch.bfloat16)
        for k0 in range(0, K, 4096):
            k1 = min(K, k0 + 4096)
            Wf[k0:k1] = (torch.randn(k1 - k0, Ns, generator=gw) * K ** -0.5).to(torch.bfloat16)
        sc = Wf.float().abs().amax(dim=0) / 127.0 + 1e-8                  # per-channel absmax
        for k0 in range(0, K, 4096):
            k1 = min(K, k0 + 4096)
            W[k0:k1] = torch.clamp(torch.round(Wf[k0:k1].float() / sc[None, :]), -128, 127).to(torch.int8)
        h["W"] = W
        h["sc"] = sc.contiguous()
        h["bias"] = (torch.randn(Ns, generator=gw) * 0.02).to(torch.bfloat16)
    if preset == "k0a":
        h["residual"] = torch.randn(M, Ns, generator=gw).to(torch.bfloat16)
        h["gamma"] = (1.0 + 0.02 * torch.randn(Ns, generator=gw)).contiguous()
    if preset == "k4v2":
        pos = torch.arange(M, dtype=torch.float32)[:, None]
        i = torch.arange(64, dtype=torch.float32)[None, :]
        ang = pos * torch.pow(torch.tensor(500000.0), -2.0 * i / 128.0)
        cs = torch.empty(M, 128)
        cs[:, 0::2] = torch.cos(ang)
        cs[:, 1::2] = torch.sin(ang)
        h["cos_sin"] = cs.contiguous()
    if h["X"] is not None:
        h["X"] = h["X"].contiguous().pin_memory() if torch.cuda.is_available() else h["X"].contiguous()
        h["R"] = h["R"].pin_memory() if torch.cuda.is_available() else h["R"]
    return h


def build_stage_gpu(capi, stage, h, dev, share=None, prev=None, world=1, gather=None, consume=None):
    """Device buffers + the fused plan of one stage.  With `share` (an earlier build of the same
    stage) the static operands (weights, per-column vectors, tables) are reused and only the
    per-step buffers (activations, row scales, output) are new: the second buffer set of the
    pipelined end-to-end loop."""
    import torch
    preset, M, N, K, dt = stage[:5]
    chain = len(stage) > 5 and stage[5] == "chain"
    Ns = h["W"].shape[1]
    s = {"stage": stage, "Ns": Ns, "chain": chain}
    a_k_slabs = False
    if chain:
        # A = the previous stage's output: in place on one GPU, the all-gathered K slabs otherwise
        if world == 1:
            s["X"] = prev["D"]
        elif consume is not None:      # slabs already filled by the producer's epilogue (peer stores)
            s["X"] = consume.tensor
            s["barrier"] = consume
            a_k_slabs = True
        else:
            s["X"] = torch.empty((world,) + tuple(prev["D"].shape), dtype=torch.bfloat16, device=dev)
            s["gather_from"] = prev["D"]
            a_k_slabs = True
        s["R"] = None
    else:
        s["X"] = h["X"].to(dev, non_blocking=True)
        s["R"] = h["R"].to(dev, non_blocking=True)
    s["W"] = share["W"] if share else h["W"].to(dev)
    kw = {}
    n_out = Ns
    if preset == "k1":
        kw = dict(row_scale=s["R"])
    elif preset == "k2":
        kw = dict(row_scale=s["R"], pair="swiglu", compact=True)
        n_out = Ns // 2
    elif preset == "k4v2":
        s["cos_sin"] = share["cos_sin"] if share else h["cos_sin"].to(dev)
        kw = dict(row_scale=s["R"], pair="rope", cos_sin=s["cos_sin"], cos_sin_period=128)
    elif preset == "k0a":
        s["residual"] = share["residual"] if share else h["residual"].to(dev)
        s["gamma"] = share["gamma"] if share else h["gamma"].to(dev)
        kw = dict(residual=s["residual"], col_scale=s["gamma"])
    elif preset == "w8a8":
        s["sc"] = share["sc"] if share else h["sc"].to(dev)
        s["bias"] = share["bias"] if share else h["bias"].to(dev)
        kw = dict(row_scale=s["R"], col_scale=s["sc"], bias=s["bias"])
    if gather is not None:             # D is this rank's slab of the symmetric gathered buffer
        s["D"] = gather.local_shard
        kw["d_peer_ptrs"] = gather.peer_slab_ptrs()
    else:
        s["D"] = torch.empty(M, n_out, dtype=torch.bfloat16, device=dev)
    s["plan"] = capi.GemmPlan(s["X"], s["W"], s["D"], a_k_slabs=a_k_slabs, **kw)
    s["flops"] = 2.0 * M * Ns * K
    s["h2d_bytes"] = 0 if chain else h["X"].numel() * h["X"].element_size() + h["R"].numel() * 4
    s["d2h_bytes"] = s["D"].numel() * 2
    s["bytes_resident"] = ((0 if chain and world == 1 else s["X"].numel() * s["X"].element_size())
                           + s["W"].numel() * s["W"].element_size()
                           + s["D"].numel() * 2)
    return s


def build_unfused(capi, s, dev):
    """Bare GEMM (identity epilogue) + the stand-alone kernel(s) the reference's unfused arm runs
    (autotune/pipeline_template.cpp.j2:771-797)."""
    import torch
    preset, M, N, K, dt = s["stage"][:5]
    Ns = s["Ns"]
    u = {}
    if dt == "s8":
        u["acc"] = torch.empty(M, Ns, dtype=torch.int32, device=dev)
        u["out"] = torch.empty(M, Ns, dtype=torch.bfloat16, device=dev)
        u["plan"] = capi.GemmPlan(s["X"], s["W"], u["acc"])
        bias_f32 = s["bias"].float()
        u["post"] = lambda: (capi.sa_dequant_w8a8(u["out"], u["acc"], s["R"], s["sc"]),
                             capi.sa_bias_add(u["out"], bias_f32))
        u["launches"] = 3
    else:
        u["out"] = torch.empty(M, Ns, dtype=torch.bfloat16, device=dev)
        u["plan"] = capi.GemmPlan(s["X"], s["W"], u["out"], a_k_slabs="gather_from" in s)
        if preset == "k1":
            u["post"] = lambda: capi.sa_scale_rows(u["out"], s["R"])
            u["launches"] = 2
        elif preset == "k2":
            u["post"] = lambda: (capi.sa_scale_rows(u["out"], s["R"]), capi.sa_swiglu(u["out"]))
            u["launches"] = 3
        elif preset == "k4v2":
            u["tmp"] = torch.empty_like(u["out"])
            u["cs_full"] = s["cos_sin"].repeat(1, Ns // 128).contiguous()
            u["post"] = lambda: (u["tmp"].copy_(u["out"]),
                                 capi.sa_rope_scaled(u["out"], u["tmp"], s["R"], u["cs_full"]))
            u["launches"] = 3
        elif preset == "k0a":
            u["post"] = lambda: capi.sa_residual_gamma(u["out"], s["residual"], s["gamma"])
            u["launches"] = 2
    return u


def time_loop(torch, fn, steps, flush=None):
    """CUDA-event time of `steps` calls on the current stream, in ms.  With `flush`, a buffer larger
    than L2 is overwritten before every step and only the steps are timed."""
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    evs = []
    for _ in range(steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs)


# ------------------------------------------------------------------------------ CPU arm
def cpu_sample(stages, seconds_target, seed):
    """Times the oracle on a row-sample of the workload; returns (tflops, rows, seconds, cores)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle as o
    o.build()
    rng = np.random.default_rng(seed)
    cores = o.num_threads()
    # bound the sample by columns too so that the widened weight panel stays small
    plans = []
    for (preset, M, N, K, dt) in [st[:5] for st in stages]:
        Nc = min(N, 4096)
        plans.append((preset, M, Nc, K, dt))
    # calibrate on 16 rows
    def run(rows):
        t = 0.0
        fl = 0.0
        for (preset, M, Nc, K, dt) in plans:
            r = min(rows, M)
            if dt == "bf16":
                A = o.f32_to_bf16(rng.standard_normal((r, K)).astype(np.float32))
                B = o.f32_to_bf16((rng.standard_normal((K, Nc)) * K ** -0.5).astype(np.float32))
                R = o.compute_rstd(A)
                t0 = time.perf_counter()
                acc = o.gemm_bf16(A, B)
                if preset == "k1":
                    o.epilogue(acc, row=R)
                elif preset == "k2":
                    o.epilogue(acc, row=R, pair="swiglu", compact=True)
                elif preset == "k4v2":
                    o.epilogue(acc, row=R, pair="rope", cos_sin=o.rope_table(r, 128, 500000.0), cos_sin_period=128)
                elif preset == "k0a":
                    o.epilogue(acc, residual=o.f32_to_bf16(acc), col=np.ones(Nc, np.float32))
                t += time.perf_counter() - t0
            else:
                A = rng.integers(-127, 128, (r, K), dtype=np.int8)
                B = rng.integers(-127, 128, (K, Nc), dtype=np.int8)
                t0 = time.perf_counter()
                acc = o.gemm_s8(A, B)
                o.epilogue(acc, row=np.full(r, 0.01, np.float32), col=np.full(Nc, 0.01, np.float32),
                           bias=np.zeros(Nc, np.float32))
                t += time.perf_counter() - t0
            fl += 2.0 * r * Nc * K
        return t, fl
    t16, f16 = run(16)
    rows = int(max(16, min(max(p[1] for p in plans), 16 * seconds_target / max(t16, 1e-3))))
    rows = (rows // 4) * 4
    t, fl = run(rows)
    return fl / t / 1e12, rows, t, cores, [p[2] for p in plans]


def run_reference_arm(args, stages):
    """`--impl reference`: the reference's path on the host cores.  The reference itself is SYCL
    for Intel Xe with no host implementation, so this is the CPU oracle (a port of its formulas)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = args.steps, args.warmup
    per_step = max(0.5, min(4.0, 120.0 / max(1, steps + warm)))
    vals = []
    rows = cores = None
    cols = None
    t_all = 0.0
    for i in range(warm + steps):
        v, rows, t, cores, cols = cpu_sample(stages, per_step, seed=i)
        if i >= warm:
            vals.append(v)
            t_all += t
    value = sum(vals) / len(vals)
    sample = f"{rows} rows x {cols} columns x full K per step of: {DESCR[args.workload]}"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": 1000.0 * t_all / len(vals),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8" if stages[0][4] == "s8" else "bf16", "data": "synthetic",
        "config": {"workload": DESCR[args.workload], "arm": "CPU oracle (port) on host cores, OpenMP"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="k2", choices=sorted(WORKLOADS))
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N>1, chained stages: all-gather fused into the producer's epilogue "
                         "(peer stores) or a separate ncclAllGather")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="single-GPU runs only: run ONE rank's column shard of an N-way split alone "
                         "(the kernel a rank of --gpus N launches), e.g. to profile it; not a job figure")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-unfused", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    stages = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, stages)
        return

    import torch
    import xefuse_loader
    xf = xefuse_loader.load()
    capi = xf.capi
    if not os.path.exists(capi.LIB_PATH):
        xf.build()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the fused path has no CPU fallback "
                         "(use --impl reference for the CPU arm)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    peaks = load_peaks()
    l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size

    shape_world = world
    if args.shard_of > 1:
        if world != 1 or any(len(st) > 5 and st[5] == "chain" for st in stages):
            raise SystemExit("bench.py --shard-of needs a single process and a workload without a gather")
        shape_world = args.shard_of
    host = [gen_stage_host(st, rank, shape_world, seed=2024 + i) for i, st in enumerate(stages)]

    def build_set(share_from=None):
        """One set of per-step buffers + plans for all stages.  When a stage feeds a chained
        consumer on several GPUs, its output goes to a symmetric gathered buffer: fused into the
        producer's epilogue (--gather fused) or by ncclAllGather afterwards (--gather nccl)."""
        out, pending = [], None
        for i, (st, h) in enumerate(zip(stages, host)):
            nxt_chain = i + 1 < len(stages) and len(stages[i + 1]) > 5
            gather = None
            if nxt_chain and world > 1 and args.gather == "fused":
                n_out = (st[2] // world) // (2 if st[0] == "k2" else 1)
                gather = xf.sharding.GatherBuffer(dist, st[1], n_out, torch.bfloat16, dev)
            out.append(build_stage_gpu(capi, st, h, dev, share=share_from[i] if share_from else None,
                                       prev=out[-1] if out else None, world=world, gather=gather, consume=pending))
            pending = gather
        return out

    gpu = build_set()
    torch.cuda.synchronize()
    resident = sum(s["bytes_resident"] for s in gpu)
    # Small workloads would run from L2 if the same buffers were reused every step: rotate over
    # enough independent copies of the whole working set that a copy's lines have been evicted
    # (more than 2.5 x L2 of other traffic) before it is used again.  No flush kernel is needed and
    # the steps stay back to back.
    flush = None
    rot = [gpu]
    if resident < 2 * l2_bytes:
        copies = int(math.ceil(2.5 * l2_bytes / max(resident, 1))) + 1
        rot += [build_set() for _ in range(copies - 1)]
        torch.cuda.synchronize()
    flops_rank = sum(s["flops"] for s in gpu)
    flops_total = flops_rank * world

    def run_stages(stage_list, stream=None):
        for s in stage_list:
            if "gather_from" in s:   # the one exchange of the path: output shards -> K slabs
                xf.sharding.all_gather_shards(dist, s["gather_from"], s["X"])
            if "barrier" in s:       # slabs were written by the producers' epilogues: wait for all
                s["barrier"].barrier()
            s["plan"].run(stream)

    turn = [0]

    def step():
        run_stages(rot[turn[0] % len(rot)])
        turn[0] += 1

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    if not uuid.startswith("GPU-"):
        uuid = "GPU-" + uuid
    sampler = ClockSampler(uuid)
    sampler.start()
    time.sleep(0.15)
    # EXACTLY `steps` steps are timed.  That region is milliseconds long, shorter than one
    # nvidia-smi sample, so the same step is then repeated untimed for about half a second and the
    # SM clock is read over that window; throttle reasons are collected over the whole run.
    t0w = time.time()
    ms = time_loop(torch, step, args.steps, flush)
    barrier()
    t1w = time.time()
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    for g in rot:
        for s in g:
            if s["plan"].device_status() != 0:
                raise SystemExit("bench.py: a kernel reported a bounded-wait timeout")
    value = flops_total * args.steps / (ms * 1e-3) / 1e12
    ms_per_step = ms / args.steps
    # the same number of repeats on every rank (ms is the max over ranks): stages may hold collectives
    load_steps = max(args.steps, min(20000, int(0.5 / max(ms_per_step * 1e-3, 1e-6))))
    tl0 = time.time()
    for i in range(load_steps):
        step()
        if i % 64 == 63:
            torch.cuda.synchronize()
    barrier()
    tl1 = time.time()

    # ---- end to end through the C ABI with host buffers: every step copies its activations and
    # row scales from pinned host memory and reads its whole output back.  Two device buffer sets
    # and three streams (copy-in, compute, copy-out) let step i+1's upload and step i-1's read-back
    # overlap step i's kernels, as a serving loop would; weights stay resident.
    gpu2 = build_set(share_from=gpu)
    sets = [gpu, gpu2]
    outs = [[torch.empty(s["D"].shape, dtype=torch.bfloat16).pin_memory() for s in gpu] for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_comp = torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_k = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    # From 4 ranks up the replicated activations are uploaded in row shards and exchanged over
    # NVLink: at 2 ranks the read-back of the output is the longer PCIe transfer either way and the
    # gather kernel only takes SMs from the persistent GEMM (measured: 813 vs 713 TFLOP/s).
    shard_upload = world >= 4 and all(s["chain"] or s["X"].shape[0] % world == 0 for s in gpu)

    def e2e_loop(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_k[b])            # the kernels that read this buffer set are done
                for s, h in zip(sets[b], host):
                    if not s["chain"]:
                        if shard_upload:
                            # replicated activations: each rank uploads 1/world of the rows over its
                            # own PCIe link and the ranks exchange them over NVLink (in-place gather)
                            m = s["X"].shape[0] // world
                            mine = s["X"][rank * m:(rank + 1) * m]
                            mine.copy_(h["X"][rank * m:(rank + 1) * m], non_blocking=True)
                            dist.all_gather_into_tensor(s["X"], mine)
                        else:
                            s["X"].copy_(h["X"], non_blocking=True)
                        s["R"].copy_(h["R"], non_blocking=True)
                ev_in[b].record(s_in)
            s_comp.wait_event(ev_in[b])
            s_comp.wait_event(ev_out[b])            # the previous read-back of this output is done
            run_stages(sets[b], s_comp.cuda_stream)
            ev_k[b].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[b])
                for s, o in zip(sets[b], outs[b]):
                    o.copy_(s["D"], non_blocking=True)
                ev_out[b].record(s_out)
        s_comp.wait_stream(s_in)
        s_comp.wait_stream(s_out)

    e2e_loop(4)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_comp)
    e2e_loop(args.steps)
    e1.record(s_comp)
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1)
    barrier()
    if dist is not None:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    # bytes that cross PCIe per step, all ranks together
    h2d_job = d2h_job = 0
    for s in gpu:
        d2h_job += s["d2h_bytes"] * world                       # every rank reads its own shard back
        if not s["chain"]:
            x_bytes = s["X"].numel() * s["X"].element_size()
            h2d_job += (x_bytes if shard_upload else x_bytes * world) + (s["h2d_bytes"] - x_bytes) * world
    e2e = {"value": flops_total * args.steps / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": int(h2d_job), "d2h_bytes_per_step": int(d2h_job),
           "ms_per_step": ms_e2e / args.steps,
           "how": "double-buffered: H2D of step i+1 and D2H of step i-1 overlap the kernels of step i; "
                  "bytes are whole-job totals over all ranks"
                  + ("; each rank uploads 1/N of the replicated activation rows and the ranks "
                     "all-gather them over NVLink" if shard_upload else "")}
    del gpu2, sets

    # ---- unfused baseline: bare GEMM + stand-alone kernel(s)
    unfused = None
    if not args.no_unfused:
        us_rot = [[build_unfused(capi, s, dev) for s in g] for g in rot]
        us = us_rot[0]

        def unfused_step():
            k = turn[0] % len(rot)
            turn[0] += 1
            for u, s in zip(us_rot[k], rot[k]):
                if "gather_from" in s:   # same exchange as the fused arm
                    xf.sharding.all_gather_shards(dist, s["gather_from"], s["X"])
                if "barrier" in s:       # unfused arm: gather the fused producer's slab with NCCL
                    xf.sharding.all_gather_shards(dist, s["barrier"].local_shard, s["X"])
                u["plan"].run()
                u["post"]()

        for _ in range(3):
            unfused_step()
        barrier()
        ms_u = time_loop(torch, unfused_step, args.steps, flush)
        barrier()
        if dist is not None:
            t = torch.tensor([ms_u], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_u = float(t.item())
        v_u = flops_total * args.steps / (ms_u * 1e-3) / 1e12
        unfused = {"value": v_u, "unit": "TFLOP/s", "ms_per_step": ms_u / args.steps,
                   "fused_speedup": value / v_u, "launches_per_step": sum(u["launches"] for u in us)}
        del us, us_rot
    clocks = sampler.stop(t0w, time.time(), load_window=(tl0 + 0.1, tl1))

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    is_s8 = stages[0][4] == "s8"
    peak = peaks["bf16"] * (2.0 if is_s8 else 1.0)
    achieved = flops_rank / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": None,
                "peak_source": ("2 x measured bf16 burst (int8 runs at twice the bf16 rate; no int8 peak was measured)"
                                if is_s8 else f"bf16 burst, {peaks['src']}"),
                "frac_of_sustained": achieved / (peaks["bf16_sustained"] * (2.0 if is_s8 else 1.0))
                if peaks.get("bf16_sustained") else None,
                "frac_of_nominal": achieved / (4500.0 if is_s8 else 2250.0),
                "kernel": ",".join(sorted({s["plan"].kernel_name for s in gpu}))}
    if world == 1:
        roofline["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload)

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        v, rows, t, cores, cols = cpu_sample(stages, args.cpu_seconds, seed=0)
        cpu_baseline = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                        "sample": f"{rows} rows x {cols} columns x full K of the workload, {t:.1f} s of CPU time"}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "s8" if is_s8 else "bf16", "data": "synthetic",
        "config": {"workload": DESCR[args.workload],
                   "sharding": ((f"ONE rank's shard of a {shape_world}-way column split, run alone; value is this GPU's rate; "
                                 if shape_world != world else "") +
                                f"weight columns N split {shape_world}-way, activations and row scales replicated, no collective inside a stage"
                                + ((f"; gate/up output shards all-gathered into K slabs for the down projection "
                                    f"({'peer stores from the epilogue' if args.gather == 'fused' else 'ncclAllGather'})")
                                   if world > 1 and any(s["chain"] for s in gpu) else "")),
                   "l2": (f"steps rotate over {len(rot)} independent copies of the working set "
                          f"({(resident * len(rot)) >> 20} MiB in all > 2.5 x L2 {l2_bytes >> 20} MiB), no flush"
                          if len(rot) > 1 else
                          f"resident inputs+outputs {resident >> 20} MiB > L2 {l2_bytes >> 20} MiB, no flush"),
                   "kernels": [s["plan"].kernel_name for s in gpu]},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "unfused": unfused,
        "gpu_launches": args.steps * len(gpu), "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
