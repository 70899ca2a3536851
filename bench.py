#!/usr/bin/env python
"""Benchmark of the fused GEMM + epilogue path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload k2] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input: one fused launch (the
`pipeline` workload: its four launches).  Default workload: k2 = GEMM + RMSNorm row-scale + SwiGLU
at the Llama-3-8B FFN gate/up shape (M=4096 tokens, K=4096, N=28672 interleaved gate/up columns,
output [4096,14336] bf16).  With N GPUs the weight columns are sharded N-ways (activations and
per-row scales replicated, nothing exchanged inside a stage), so total work is fixed: strong
scaling.  Prints ONE JSON line on rank 0.

  value       whole-job TFLOP/s (2*M*N*K per GEMM), inputs resident in HBM, CUDA-event timed,
              max over ranks
  value_sustained
              the same step repeated back to back for about half a second (the part then sits on
              its power cap), with the SM clock sampled over that window
  e2e         the same metric through the C ABI with HOST buffers: every step copies the step's
              activations + row scales host->device from pinned memory and the output device->host
  roofline    tensor-core bound: achieved 2MNK / average launch time against the measured bf16
              peak; int8 against an int8 peak measured in the same run
  all_configs (1 GPU, default workload) the other BASELINE configurations, device-timed, with
              their unfused arm
  pipeline    (N > 1, default workload) the Llama-3-70B layer chain, whose gate/up -> down hand-off
              is the path's one collective: all-gather fused into the producer's epilogue (peer
              stores) and as a separate ncclAllGather, plus a bit-for-bit check of one against
              the other
  cpu_baseline / --impl reference
              the CPU oracle (a port of the reference's formulas; the reference has no CPU or CUDA
              implementation of its own) timed on the host cores on a bounded row-sample
"""
import argparse
import json
import math
import os
import re
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
    "k0a": [("k0a", 8192, 8192, 8192, "bf16")],          # the O-projection stage of the chain, alone
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
    "k0a": "k0a GEMM+residual+gamma Llama-3-70B O-proj M=8192 K=8192 N=8192 bf16, residual bf16 [8192,8192]",
    "rstd_quant": "RMSNorm + per-token int8 quantisation producer (compute_rstd_and_quantize) over bf16 [8192,8192]",
    "pipeline": "Llama-3-70B layer GEMM chain M=8192: QKV k4v2 (K=8192,N=10240), O k0a (8192,8192), "
                "gate/up k2 (K=8192,N=57344), down k0a (K=28672,N=8192)",
}
OTHER_CONFIGS = ["k1", "k4v2_q", "k4v2_kv", "w8a8", "pipeline"]


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16": d["bf16_tflops"], "bf16_sustained": d.get("bf16_tflops_sustained"),
                "hbm": d["hbm_gbs"], "src": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "src": "fallback"}


def load_traffic():
    """DRAM bytes per launch of each workload's kernel from the profiler summaries: the one table of
    the form `| workload | dram read B | dram write B | ...` in profiles/dram_traffic.md."""
    out = {}
    p = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(p):
        return out
    for line in open(p):
        m = re.match(r"\|\s*(\w+)\s*\|\s*([\d_,]+)\s*\|\s*([\d_,]+)\s*\|", line)
        if m:
            out[m.group(1)] = int(re.sub(r"[_,]", "", m.group(2))) + int(re.sub(r"[_,]", "", m.group(3)))
    return out


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

    def median_sm(self, t0, t1):
        v = []
        for ts, l in list(self.lines):
            f = [x.strip() for x in l.split(",")]
            if t0 <= ts <= t1 and len(f) >= 6 and f[0].isdigit():
                v.append(int(f[0]))
        v.sort()
        return (v[len(v) // 2], len(v)) if v else (None, 0)

    def stop(self, load_window=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = [[x.strip() for x in l.split(",")] for _, l in self.lines
                if l and l.split(",")[0].strip().isdigit() and len(l.split(",")) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        sm, nload = (None, 0)
        if load_window is not None:
            sm, nload = self.median_sm(*load_window)
        if sm is None:
            s = sorted(int(r[0]) for r in rows)
            sm = s[len(s) // 2]
        return {"sm_mhz": sm, "sm_max_mhz": int(rows[0][1]), "reasons": reasons,
                "samples": len(rows), "load_samples": nload,
                "how": "sm_mhz = median over the sustained repeat of the timed step; reasons over the whole run"}


# ------------------------------------------------------------------------------ synthetic inputs
def gen_stage(stage, rank, world, seed, dev, host_x=True):
    """Seeded synthetic tensors of one stage for this rank's column shard.  Activations and row
    scales are made on the host (pinned: the end-to-end arm copies them every step) unless
    host_x is False; weights, per-column vectors and tables are made on the device."""
    import torch
    preset, M, N, K, dt = stage[:5]
    chain = len(stage) > 5 and stage[5] == "chain"
    assert N % world == 0
    Ns = N // world
    g = torch.Generator().manual_seed(seed)
    gd = torch.Generator(device=dev).manual_seed(seed * 7919 + 13 * rank + 1)   # per-shard weight stream
    h = {"X": None, "R": None}

    def randn_dev(*shape):
        return torch.randn(*shape, generator=gd, device=dev, dtype=torch.float32)

    def bounded_rows(fn, rows):      # weights in row blocks: bounded fp32 temporaries
        for k0 in range(0, rows, 4096):
            fn(k0, min(rows, k0 + 4096))

    if dt == "bf16":
        if not chain:
            if host_x:
                X = torch.randn(M, K, generator=g, dtype=torch.float32)
            else:
                X = torch.randn(M, K, generator=torch.Generator(device=dev).manual_seed(seed), device=dev)
            h["R"] = torch.rsqrt((X * X).mean(dim=1) + 1e-6).contiguous()    # fp32
            h["X"] = X.to(torch.bfloat16)
        W = torch.empty(K, Ns, dtype=torch.bfloat16, device=dev)
        bounded_rows(lambda a, b: W[a:b].copy_((randn_dev(b - a, Ns) * K ** -0.5).to(torch.bfloat16)), K)
        h["W"] = W
    else:
        gx = g if host_x else torch.Generator(device=dev).manual_seed(seed)
        X = torch.randn(M, K, generator=gx, dtype=torch.float32,
                        device="cpu" if host_x else dev).to(torch.bfloat16).float()
        st = X.abs().amax(dim=1) / 127.0 + 1e-8                          # per-token absmax
        h["X"] = torch.clamp(torch.round(X / st[:, None]), -128, 127).to(torch.int8)
        h["R"] = st.contiguous()
        Wf = torch.empty(K, Ns, dtype=torch.bfloat16, device=dev)
        bounded_rows(lambda a, b: Wf[a:b].copy_((randn_dev(b - a, Ns) * K ** -0.5).to(torch.bfloat16)), K)
        sc = Wf.float().abs().amax(dim=0) / 127.0 + 1e-8                  # per-channel absmax
        W = torch.empty(K, Ns, dtype=torch.int8, device=dev)
        bounded_rows(lambda a, b: W[a:b].copy_(
            torch.clamp(torch.round(Wf[a:b].float() / sc[None, :]), -128, 127).to(torch.int8)), K)
        del Wf
        h["W"] = W
        h["sc"] = sc.contiguous()
        h["bias"] = (randn_dev(Ns) * 0.02).to(torch.bfloat16)
    if preset == "k0a":
        h["residual"] = randn_dev(M, Ns).to(torch.bfloat16)
        h["gamma"] = (1.0 + 0.02 * randn_dev(Ns)).contiguous()
    if preset == "k4v2":
        pos = torch.arange(M, dtype=torch.float32, device=dev)[:, None]
        i = torch.arange(64, dtype=torch.float32, device=dev)[None, :]
        ang = pos * torch.pow(torch.tensor(500000.0, device=dev), -2.0 * i / 128.0)
        cs = torch.empty(M, 128, device=dev)
        cs[:, 0::2] = torch.cos(ang)
        cs[:, 1::2] = torch.sin(ang)
        h["cos_sin"] = cs.contiguous()
    if h["X"] is not None and host_x:
        h["X"] = h["X"].contiguous().pin_memory()
        h["R"] = h["R"].pin_memory()
    return h


def build_stage_gpu(capi, stage, h, dev, share=None, prev=None, world=1, gather=None, consume=None,
                    x_buffer=None):
    """Device buffers + the fused plan of one stage.  With `share` (an earlier build of the same
    stage) the static operands (weights, per-column vectors, tables) are reused and only the
    per-step buffers (activations, row scales, output) are new."""
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
    elif x_buffer is not None:         # activations live in a buffer the caller provides (peer-mapped)
        s["X"] = x_buffer
        s["X"].copy_(h["X"], non_blocking=True)
        s["R"] = h["R"].to(dev, non_blocking=True)
    else:
        s["X"] = h["X"].to(dev, non_blocking=True) if h["X"].device != dev or share else h["X"]
        s["R"] = h["R"].to(dev, non_blocking=True) if h["R"].device != dev or share else h["R"]
        if share and s["X"].data_ptr() == h["X"].data_ptr():   # device-made inputs: a private copy per set
            s["X"], s["R"] = h["X"].clone(), h["R"].clone()
    s["W"] = share["W"] if share else h["W"]
    kw = {}
    n_out = Ns
    if preset == "k1":
        kw = dict(row_scale=s["R"])
    elif preset == "k2":
        kw = dict(row_scale=s["R"], pair="swiglu", compact=True)
        n_out = Ns // 2
    elif preset == "k4v2":
        s["cos_sin"] = h["cos_sin"]
        kw = dict(row_scale=s["R"], pair="rope", cos_sin=s["cos_sin"], cos_sin_period=128)
    elif preset == "k0a":
        s["residual"], s["gamma"] = h["residual"], h["gamma"]
        kw = dict(residual=s["residual"], col_scale=s["gamma"])
    elif preset == "w8a8":
        s["sc"], s["bias"] = h["sc"], h["bias"]
        kw = dict(row_scale=s["R"], col_scale=s["sc"], bias=s["bias"])
    if gather is not None:             # D is this rank's slab of the symmetric gathered buffer
        s["D"] = gather.local_shard
        kw["d_peer_ptrs"] = gather.peer_slab_ptrs()
    else:
        s["D"] = torch.empty(M, n_out, dtype=torch.bfloat16, device=dev)
    s["plan"] = capi.GemmPlan(s["X"], s["W"], s["D"], a_k_slabs=a_k_slabs, **kw)
    s["flops"] = 2.0 * M * Ns * K
    s["h2d_bytes"] = 0 if chain else s["X"].numel() * s["X"].element_size() + s["R"].numel() * 4
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
        u["plan"] = capi.GemmPlan(s["X"], s["W"], u["out"], a_k_slabs="gather_from" in s or "barrier" in s)
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


def time_loop(torch, fn, steps):
    """CUDA-event time of `steps` back-to-back calls on the current stream, in ms."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


# ------------------------------------------------------------------------------ one workload on the GPU(s)
class Workload:
    """Buffers, plans and timed loops of one workload on this rank."""

    def __init__(self, ctx, name, gather="fused", shard_of=0, host_x=True):
        import torch
        self.ctx, self.name, self.gather = ctx, name, gather
        self.torch = torch
        self.stages = WORKLOADS[name]
        self.world = ctx["world"]
        shape_world = self.world
        if shard_of > 1:
            if self.world != 1 or any(len(st) > 5 for st in self.stages):
                raise SystemExit("bench.py --shard-of needs a single process and a workload without a gather")
            shape_world = shard_of
        self.shape_world = shape_world
        dev = ctx["dev"]
        self.host = [gen_stage(st, ctx["rank"], shape_world, 2024 + i, dev, host_x=host_x)
                     for i, st in enumerate(self.stages)]
        self.gpu = self.build_set()
        torch.cuda.synchronize()
        self.resident = sum(s["bytes_resident"] for s in self.gpu)
        # Small workloads would run from L2 if the same buffers were reused every step: rotate over
        # enough independent copies of the per-step buffers AND weights that a copy's lines have been
        # evicted (more than 2.5 x L2 of other traffic) before it is used again.  No flush kernel is
        # needed and the steps stay back to back.
        self.rot = [self.gpu]
        if self.resident < 2 * ctx["l2_bytes"]:
            copies = int(math.ceil(2.5 * ctx["l2_bytes"] / max(self.resident, 1))) + 1
            for c in range(copies - 1):
                self.rot.append(self.build_set(fresh_weights=True))
            torch.cuda.synchronize()
        self.flops_rank = sum(s["flops"] for s in self.gpu)
        self.flops_total = self.flops_rank * self.world
        self.turn = 0

    def build_set(self, share_from=None, fresh_weights=False, x_alloc=None):
        """One set of per-step buffers + plans for all stages.  When a stage feeds a chained
        consumer on several GPUs, its output goes to a symmetric gathered buffer: fused into the
        producer's epilogue (gather == "fused") or by ncclAllGather afterwards ("nccl")."""
        ctx, torch = self.ctx, self.torch
        xf, capi, dist, dev = ctx["xf"], ctx["capi"], ctx["dist"], ctx["dev"]
        out, pending = [], None
        for i, (st, h) in enumerate(zip(self.stages, self.host)):
            if fresh_weights:      # an independent copy of every operand of the stage
                h = {k: (v.clone() if hasattr(v, "clone") and v is not None and v.device == dev else v)
                     for k, v in h.items()}
            nxt_chain = i + 1 < len(self.stages) and len(self.stages[i + 1]) > 5
            gather = None
            if nxt_chain and self.world > 1 and self.gather == "fused":
                n_out = (st[2] // self.world) // (2 if st[0] == "k2" else 1)
                gather = xf.sharding.GatherBuffer(dist, st[1], n_out, torch.bfloat16, dev)
            xb = x_alloc(h["X"]) if (x_alloc is not None and len(st) <= 5) else None
            out.append(build_stage_gpu(capi, st, h, dev, share=share_from[i] if share_from else None,
                                       prev=out[-1] if out else None, world=self.world, gather=gather,
                                       consume=pending, x_buffer=xb))
            pending = gather
        return out

    def run_stages(self, stage_list, stream=None):
        xf, dist = self.ctx["xf"], self.ctx["dist"]
        for s in stage_list:
            if "gather_from" in s:   # the one exchange of the path: output shards -> K slabs
                xf.sharding.all_gather_shards(dist, s["gather_from"], s["X"])
            if "barrier" in s:       # slabs were written by the producers' epilogues: wait for all
                s["barrier"].barrier()
            s["plan"].run(stream)

    def step(self):
        self.run_stages(self.rot[self.turn % len(self.rot)])
        self.turn += 1

    def max_over_ranks(self, ms):
        dist = self.ctx["dist"]
        if dist is None:
            return ms
        t = self.torch.tensor([ms], device=self.ctx["dev"])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def check_status(self):
        for g in self.rot:
            for s in g:
                if s["plan"].device_status() != 0:
                    raise SystemExit("bench.py: a kernel reported a bounded-wait timeout")

    def graph_of(self, n):
        """A CUDA graph of `n` consecutive steps of this rank (kernels only, no collective): a step
        of a small workload lasts 20-90 us, the order of what a launch through Python costs, so its
        steps are replayed from a graph instead of being launched one by one."""
        torch = self.torch
        s = torch.cuda.Stream(self.ctx["dev"])
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            self.step()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                for _ in range(n):
                    self.step()
        torch.cuda.synchronize()
        return g

    def small(self):
        # short steps without a collective are replayed from a CUDA graph (on every rank alike), so
        # that what is timed is the kernels back to back and not the host's launch calls
        return len(self.rot) > 1 and not any(s["chain"] for s in self.gpu)

    def timed(self, steps, warmup):
        """(TFLOP/s whole job, ms per step): EXACTLY `steps` steps between two barriers."""
        barrier = self.ctx["barrier"]
        for _ in range(warmup):
            self.step()
        barrier()
        if self.small():
            g = self.graph_of(steps)
            g.replay()                       # one untimed replay: graph upload
            barrier()
            ms = time_loop(self.torch, g.replay, 1)
            self.launch_mode = "CUDA graph of the timed steps"
        else:
            ms = time_loop(self.torch, self.step, steps)
            self.launch_mode = "one launch call per kernel"
        barrier()
        ms = self.max_over_ranks(ms)
        self.check_status()
        return self.flops_total * steps / (ms * 1e-3) / 1e12, ms / steps

    def step_times(self, steps):
        """A separate pass of `steps` steps with an event pair around EACH step (max over ranks per
        step): best and median ms per step, as the reference's harnesses print them."""
        torch = self.torch
        self.ctx["barrier"]()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            self.step()
            ev[i + 1].record()
        torch.cuda.synchronize()
        t = torch.tensor([ev[i].elapsed_time(ev[i + 1]) for i in range(steps)], device=self.ctx["dev"])
        if self.ctx["dist"] is not None:
            self.ctx["dist"].all_reduce(t, op=self.ctx["dist"].ReduceOp.MAX)
        t = sorted(t.tolist())
        return {"best_ms": t[0], "median_ms": t[len(t) // 2], "worst_ms": t[-1], "n": steps,
                "how": "one CUDA-event pair per step in a pass of its own, max over ranks per step"}

    def sustained(self, ms_per_step, seconds=0.5, min_steps=0):
        """The same step back to back for about `seconds`: (TFLOP/s, ms per step, wall window)."""
        barrier = self.ctx["barrier"]
        n = max(min_steps, min(20000, int(seconds / max(ms_per_step * 1e-3, 1e-6))))
        barrier()
        if self.small():
            per = 200
            g = self.graph_of(per)
            reps = max(1, n // per)
            n = reps * per
            g.replay()
            barrier()
            t0 = time.time()
            ms = time_loop(self.torch, g.replay, reps)
            t1 = time.time()
        else:
            t0 = time.time()
            ms = time_loop(self.torch, self.step, n)
            t1 = time.time()
        barrier()
        ms = self.max_over_ranks(ms)
        return self.flops_total * n / (ms * 1e-3) / 1e12, ms / n, (t0 + 0.1, t1), n

    def kernels(self):
        return [s["plan"].kernel_name for s in self.gpu]

    # ---- end to end through the C ABI with host buffers: every step copies its activations and
    # row scales from pinned host memory and reads its whole output back.  Two device buffer sets
    # and three streams (copy-in, compute, copy-out) let step i+1's upload and step i-1's read-back
    # overlap step i's kernels, as a serving loop would; weights stay resident.
    def e2e(self, steps, exchange="copy"):
        torch, ctx = self.torch, self.ctx
        dev, dist, world, rank = ctx["dev"], ctx["dist"], self.world, ctx["rank"]
        # From 4 ranks up the replicated activations are uploaded in row shards (each rank 1/N of
        # the rows over its own PCIe link) and exchanged over NVLink: at 2 ranks the read-back of
        # the output is the longer PCIe transfer either way.
        shard_upload = world >= 4 and all(len(st) > 5 or st[1] % world == 0 for st in self.stages)
        peer_push = shard_upload and exchange == "copy"
        handles = []

        def sym_alloc(like):           # activations in symmetric (peer-mapped) memory
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(tuple(like.shape), dtype=like.dtype, device=dev)
            hdl = symm.rendezvous(t, group=dist.group.WORLD)
            handles.append((t, hdl))
            return t

        if peer_push:
            sets = [self.build_set(share_from=self.gpu, x_alloc=sym_alloc) for _ in range(2)]
        else:
            sets = [self.gpu, self.build_set(share_from=self.gpu)]
        gpu = sets[0]
        peers = {}                     # X buffer -> views of the same buffer on every other rank
        for t, hdl in handles:
            peers[t.data_ptr()] = (hdl, [hdl.get_buffer(p, tuple(t.shape), t.dtype) for p in range(world) if p != rank])
        outs = [[torch.empty(s["D"].shape, dtype=torch.bfloat16).pin_memory() for s in gpu] for _ in range(2)]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        s_comp = torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_k = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        host = self.host

        def upload(b, do_h2d=True, do_xchg=True):
            for s, h in zip(sets[b], host):
                if s["chain"]:
                    continue
                if shard_upload:
                    m = s["X"].shape[0] // world
                    mine = s["X"][rank * m:(rank + 1) * m]
                    if peer_push:
                        hdl, views = peers[s["X"].data_ptr()]
                        if do_xchg:
                            hdl.barrier(channel=0)      # every rank's kernels that read this set are done
                        if do_h2d:
                            mine.copy_(h["X"][rank * m:(rank + 1) * m], non_blocking=True)
                        if do_xchg:
                            # copy engines push this rank's rows into the same rows of every peer's
                            # buffer; no SM kernel competes with the persistent GEMM
                            for v in views:
                                v[rank * m:(rank + 1) * m].copy_(mine, non_blocking=True)
                            hdl.barrier(channel=1)      # all rows of the local buffer have landed
                    else:
                        if do_h2d:
                            mine.copy_(h["X"][rank * m:(rank + 1) * m], non_blocking=True)
                        if do_xchg:
                            dist.all_gather_into_tensor(s["X"], mine)
                elif do_h2d:
                    s["X"].copy_(h["X"], non_blocking=True)
                if do_h2d:
                    s["R"].copy_(h["R"], non_blocking=True)

        def loop(n):
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_k[b])            # the kernels that read this buffer set are done
                    upload(b)
                    ev_in[b].record(s_in)
                s_comp.wait_event(ev_in[b])
                s_comp.wait_event(ev_out[b])            # the previous read-back of this output is done
                self.run_stages(sets[b], s_comp.cuda_stream)
                ev_k[b].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k[b])
                    for s, o in zip(sets[b], outs[b]):
                        o.copy_(s["D"], non_blocking=True)
                    ev_out[b].record(s_out)
            s_comp.wait_stream(s_in)
            s_comp.wait_stream(s_out)

        def timed_on(stream, fn, n):
            ctx["barrier"]()
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                a.record(stream)
                for i in range(n):
                    fn(i & 1)
                z.record(stream)
            torch.cuda.synchronize()
            return self.max_over_ranks(a.elapsed_time(z)) / n

        loop(4)
        ctx["barrier"]()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s_comp)
        loop(steps)
        e1.record(s_comp)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        ctx["barrier"]()
        ms = self.max_over_ranks(ms)
        # each phase of a step alone, back to back on its own stream (max over ranks)
        split = {"h2d": timed_on(s_in, lambda b: upload(b, do_xchg=False), steps),
                 "kernels": timed_on(s_comp, lambda b: self.run_stages(sets[b], s_comp.cuda_stream), steps),
                 "d2h": timed_on(s_out, lambda b: [o.copy_(s["D"], non_blocking=True)
                                                   for s, o in zip(sets[b], outs[b])], steps)}
        if shard_upload:
            split["exchange"] = timed_on(s_in, lambda b: upload(b, do_h2d=False), steps)
        h2d_job = d2h_job = 0          # bytes that cross PCIe per step, all ranks together
        for s in gpu:
            d2h_job += s["d2h_bytes"] * world
            if not s["chain"]:
                x_bytes = s["X"].numel() * s["X"].element_size()
                h2d_job += (x_bytes if shard_upload else x_bytes * world) + (s["h2d_bytes"] - x_bytes) * world
        return {"value": self.flops_total * steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(h2d_job), "d2h_bytes_per_step": int(d2h_job),
                "ms_per_step": ms / steps, "phase_ms_alone": split,
                "how": "double-buffered: H2D of step i+1 and D2H of step i-1 overlap the kernels of step i; "
                       "bytes are whole-job totals over all ranks; phase_ms_alone = each phase run by itself"
                       + ("; each rank uploads 1/N of the replicated activation rows and "
                          + ("pushes them into every peer's buffer with copy-engine peer copies between two "
                             "stream-ordered barriers" if peer_push else "the ranks all-gather them with NCCL")
                          if shard_upload else "")}

    # ---- unfused baseline: bare GEMM + stand-alone kernel(s)
    def unfused(self, steps, fused_value):
        ctx = self.ctx
        xf, capi, dist, dev = ctx["xf"], ctx["capi"], ctx["dist"], ctx["dev"]
        us_rot = [[build_unfused(capi, s, dev) for s in g] for g in self.rot]

        def ustep():
            k = self.turn % len(self.rot)
            self.turn += 1
            for u, s in zip(us_rot[k], self.rot[k]):
                if "gather_from" in s:   # same exchange as the fused arm
                    xf.sharding.all_gather_shards(dist, s["gather_from"], s["X"])
                if "barrier" in s:       # unfused arm: gather the fused producer's slab with NCCL
                    xf.sharding.all_gather_shards(dist, s["barrier"].local_shard, s["X"])
                u["plan"].run()
                u["post"]()

        for _ in range(3):
            ustep()
        ctx["barrier"]()
        if self.small():                     # replayed from a graph like the fused steps
            torch = self.torch
            st = torch.cuda.Stream(dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(st):
                ustep()
                torch.cuda.synchronize()
                with torch.cuda.graph(g, stream=st):
                    for _ in range(steps):
                        ustep()
            torch.cuda.synchronize()
            g.replay()
            ctx["barrier"]()
            ms = time_loop(torch, g.replay, 1)
        else:
            ms = time_loop(self.torch, ustep, steps)
        ctx["barrier"]()
        ms = self.max_over_ranks(ms)
        v = self.flops_total * steps / (ms * 1e-3) / 1e12
        return {"value": v, "unit": "TFLOP/s", "ms_per_step": ms / steps, "fused_speedup": fused_value / v,
                "launches_per_step": sum(u["launches"] for u in us_rot[0])}

    def l2_note(self):
        l2 = self.ctx["l2_bytes"]
        if len(self.rot) > 1:
            return (f"steps rotate over {len(self.rot)} independent copies of the working set "
                    f"({(self.resident * len(self.rot)) >> 20} MiB in all > 2.5 x L2 {l2 >> 20} MiB), no flush; "
                    f"{getattr(self, 'launch_mode', '')}")
        return f"resident inputs+outputs {self.resident >> 20} MiB > L2 {l2 >> 20} MiB, no flush"


def measure_int8_peak(ctx):
    """int8 tensor-core rate of this GPU on an 8192^3 problem in local memory: cuBLASLt through
    torch._int_mm (the library yardstick) and this library's bare int8 kernel (int32 output, no
    epilogue).  Best of 10 single launches, CUDA events.  TOP/s."""
    torch, capi, dev = ctx["torch"], ctx["capi"], ctx["dev"]
    n = 8192
    out = {"shape": "8192^3 int8 -> int32", "how": "best of 10 single launches, CUDA events"}
    A = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=dev)
    B = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=dev)

    def best(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        t = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            t.append(a.elapsed_time(b))
        return 2.0 * n ** 3 / (min(t) * 1e-3) / 1e12

    try:
        Bt = B.t().contiguous().t()        # column-major B: the layout cuBLASLt's int8 GEMM wants
        out["torch_int_mm"] = best(lambda: torch._int_mm(A, Bt))
    except Exception as e:                 # noqa: BLE001  (library call that may refuse the layout)
        out["torch_int_mm"] = None
        out["torch_int_mm_error"] = str(e)[:120]
    D = torch.empty((n, n), dtype=torch.int32, device=dev)
    plan = capi.GemmPlan(A, B, D)
    out["own_bare_kernel"] = best(plan.run)
    out["kernel"] = plan.kernel_name
    return out


def gather_check(ctx, steps=2):
    """N > 1: the all-gather fused into the producer's epilogue against ncclAllGather, bit for bit,
    on a small gate/up -> down chain: the gathered buffers must be identical and so must the
    consumer's outputs.  Returns "pass" or a short failure text."""
    torch, dist, dev, xf, capi = ctx["torch"], ctx["dist"], ctx["dev"], ctx["xf"], ctx["capi"]
    world, rank = ctx["world"], ctx["rank"]
    sh = xf.sharding
    M, K1, N2 = 512, 512, 512
    N1 = 2 * 256 * 2 * world
    g = torch.Generator(device=dev).manual_seed(5)            # identical on every rank: replicated inputs
    X = torch.randn(M, K1, generator=g, device=dev).to(torch.bfloat16)
    R = torch.rsqrt((X.float() ** 2).mean(dim=1) + 1e-6).contiguous()
    W1 = (torch.randn(K1, N1, generator=g, device=dev) * K1 ** -0.5).to(torch.bfloat16)
    W2 = (torch.randn(N1 // 2, N2, generator=g, device=dev) * (N1 // 2) ** -0.5).to(torch.bfloat16)
    lo, hi = sh.shard_columns(N1, world, rank, sh.stage_multiple("k2", compact=True))
    ns = (hi - lo) // 2
    W1s = W1[:, lo:hi].contiguous()
    gb = sh.GatherBuffer(dist, M, ns, torch.bfloat16, dev)
    gb.tensor.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    prod = capi.GemmPlan(X, W1s, gb.local_shard, row_scale=R, pair="swiglu", compact=True,
                         d_peer_ptrs=gb.peer_slab_ptrs())
    out_f = torch.empty(M, N2, dtype=torch.bfloat16, device=dev)
    cons_f = capi.GemmPlan(gb.tensor, W2, out_f, a_k_slabs=True)
    shard = torch.empty(M, ns, dtype=torch.bfloat16, device=dev)
    gathered = torch.zeros(world, M, ns, dtype=torch.bfloat16, device=dev)
    prod_n = capi.GemmPlan(X, W1s, shard, row_scale=R, pair="swiglu", compact=True)
    out_n = torch.empty(M, N2, dtype=torch.bfloat16, device=dev)
    cons_n = capi.GemmPlan(gathered, W2, out_n, a_k_slabs=True)
    for _ in range(steps):
        prod.run()
        gb.barrier()
        cons_f.run()
        prod_n.run()
        sh.all_gather_shards(dist, shard, gathered)
        cons_n.run()
        gb.barrier()              # nobody overwrites a slab a peer may still read
    torch.cuda.synchronize()
    ok = torch.equal(gb.tensor.view(torch.int16), gathered.view(torch.int16)) and \
        torch.equal(out_f.view(torch.int16), out_n.view(torch.int16)) and bool(out_f.float().abs().sum() > 0)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return "pass" if int(flag.item()) == 1 else "FAIL: fused gather differs from ncclAllGather on some rank"


def run_rstd_quant(ctx, args, peaks):
    """The activation-quantisation producer (kernels/compute_rstd.hpp:67-125 of the reference): one
    HBM-bound row pass, 2 bytes read + 1 byte written per element (+ 4 per row)."""
    torch, capi, dev = ctx["torch"], ctx["capi"], ctx["dev"]
    M = N = 8192
    rot = []
    for i in range(3):      # 3 x 201 MB: every step reads cold rows
        x = torch.randn(M, N, device=dev, generator=torch.Generator(device=dev).manual_seed(7 + i)).to(torch.bfloat16)
        rot.append((x, torch.empty(M, N, dtype=torch.int8, device=dev), torch.empty(M, dtype=torch.float32, device=dev)))
    turn = [0]

    def step():
        x, q, st = rot[turn[0] % len(rot)]
        turn[0] += 1
        capi.compute_rstd_and_quantize(x, q, st)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    ms = time_loop(torch, step, args.steps) / args.steps
    algo = M * N * 3 + M * 4
    gbs = algo / (ms * 1e-3) / 1e9
    line = {"metric": "rstd+quantise producer GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16->s8", "data": "synthetic",
            "config": {"workload": DESCR["rstd_quant"], "l2": "steps rotate over 3 inputs of 134 MB each, no flush"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm"], "traffic": None, "peak_source": f"STREAM-style copy, {peaks['src']}"},
            "gpu_launches": args.steps}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ CPU arm
def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample(stages, seconds_target, seed):
    """Times the oracle on a row-sample of the workload; returns (tflops, rows, seconds, cores)."""
    # all the host cores this process may use, whatever the launcher put in OMP_NUM_THREADS
    # (torch.distributed.run sets it to 1)
    os.environ["OMP_NUM_THREADS"] = str(cpu_threads())
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle as o
    o.build()
    o.set_num_threads(cpu_threads())
    rng = np.random.default_rng(seed)
    cores = o.num_threads()
    # bound the sample by columns too so that the widened weight panel stays small
    plans = []
    for (preset, M, N, K, dt) in [st[:5] for st in stages]:
        Nc = min(N, 4096)
        plans.append((preset, M, Nc, K, dt))

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
    m_max = max(p[1] for p in plans)
    rows = int(max(16, min(m_max, 16 * seconds_target / max(t16, 1e-3))))
    rows = (rows // 4) * 4
    # all rows fit the time target: widen the column sample too, up to the whole workload
    t_rows = t16 * rows / 16.0
    if rows >= m_max and t_rows < seconds_target:
        grow = seconds_target / max(t_rows, 1e-3)
        plans = [(preset, M, int(min(N, max(Nc, (int(Nc * grow) // 256) * 256))), K, dt)
                 for (preset, M, Nc, K, dt), N in zip(plans, [st[2] for st in stages])]
    t, fl = run(rows)
    return fl / t / 1e12, rows, t, cores, [p[2] for p in plans]


def cpu_library_gemm(stages, seconds_target=3.0):
    """The best CPU GEMM at hand for context: torch.matmul (oneDNN/MKL) on the same host cores, on
    the first stage's K and up to 4096 of its columns, GEMM only (no epilogue)."""
    import torch
    (_, M, N, K, dt) = stages[0][:5]
    torch.set_num_threads(cpu_threads())
    Nc, r = min(N, 4096), min(M, 1024)
    if dt == "bf16":
        A = torch.randn(r, K).to(torch.bfloat16)
        B = torch.randn(K, Nc).to(torch.bfloat16)
        fn, what = (lambda: torch.matmul(A, B)), "torch.matmul bf16"
    else:
        A = torch.randint(-127, 128, (r, K), dtype=torch.int8)
        B = torch.randint(-127, 128, (K, Nc), dtype=torch.int8)
        fn, what = (lambda: torch._int_mm(A, B)), "torch._int_mm int8"
    try:
        fn()
        n, t0 = 0, time.perf_counter()
        while n < 2 or (time.perf_counter() - t0 < seconds_target and n < 200):
            fn()
            n += 1
        t = (time.perf_counter() - t0) / n
    except Exception as e:        # a CPU build without that kernel: report it, the oracle figure stands
        return {"unavailable": f"{what} on CPU: {type(e).__name__}"}
    return {"value": 2.0 * r * Nc * K / t / 1e12, "unit": "TOP/s" if dt != "bf16" else "TFLOP/s",
            "what": f"{what}, {r} x {Nc} x {K}, GEMM only, {torch.get_num_threads()} threads"}


def run_reference_arm(args, stages):
    """`--impl reference`: the reference's path on the host cores.  The reference itself is SYCL
    for Intel Xe with no host implementation, so this is the CPU oracle (a port of its formulas),
    on every core this process may use.  Under torch.distributed.run only rank 0 works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = args.steps, args.warmup
    per_step = max(0.5, min(6.0, 120.0 / max(1, steps + warm)))   # CPU seconds of oracle work per step
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
    ap.add_argument("--workload", default="k2", choices=sorted(WORKLOADS) + ["rstd_quant"])
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N>1, chained stages: all-gather fused into the producer's epilogue "
                         "(peer stores) or a separate ncclAllGather")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="single-GPU runs only: run ONE rank's column shard of an N-way split alone "
                         "(the kernel a rank of --gpus N launches), e.g. to profile it; not a job figure")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-unfused", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer arm (profiling runs)")
    ap.add_argument("--e2e-exchange", default="copy", choices=["copy", "nccl"],
                    help="N>=4, end-to-end arm: how the row shards of the replicated activations reach "
                         "the other ranks: copy-engine peer copies (default) or an NCCL all-gather")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip all_configs (1 GPU) / pipeline + gather check (N > 1) and the int8 peak")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    stages = WORKLOADS.get(args.workload)
    if stages is None and (args.impl == "reference" or args.gpus > 1):
        raise SystemExit("bench.py: the rstd_quant workload is a single-GPU row pass of this library only")

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

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = load_peaks()
    ctx = {"torch": torch, "xf": xf, "capi": capi, "dist": dist, "dev": dev, "world": world, "rank": rank,
           "barrier": barrier, "l2_bytes": torch.cuda.get_device_properties(dev).L2_cache_size}

    if stages is None:
        run_rstd_quant(ctx, args, peaks)
        return
    wl = Workload(ctx, args.workload, gather=args.gather, shard_of=args.shard_of)
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    if not uuid.startswith("GPU-"):
        uuid = "GPU-" + uuid
    sampler = ClockSampler(uuid)
    sampler.start()
    time.sleep(0.15)
    # EXACTLY `steps` steps are timed.  That region is milliseconds long, shorter than one
    # nvidia-smi sample, so the same step is then repeated for about half a second, timed as
    # value_sustained, and the SM clock is read over that window; throttle reasons are collected
    # over the whole run.
    value, ms_per_step = wl.timed(args.steps, args.warmup)
    step_times = wl.step_times(args.steps)
    v_sus, ms_sus, load_window, n_sus = wl.sustained(ms_per_step, min_steps=args.steps)
    sm_sus, _ = sampler.median_sm(*load_window)

    e2e = None if args.no_e2e else wl.e2e(args.steps, exchange=args.e2e_exchange)
    unfused = None if args.no_unfused else wl.unfused(args.steps, value)
    is_s8 = stages[0][4] == "s8"
    kernels = wl.kernels()
    l2_note = wl.l2_note()
    flops_rank, shape_world = wl.flops_rank, wl.shape_world
    n_stage = len(wl.gpu)
    has_chain = any(s["chain"] for s in wl.gpu)
    del wl
    torch.cuda.empty_cache()

    # ---- extras: the other configurations (1 GPU) or the collective-bearing chain (N > 1)
    default_run = args.workload == "k2" and args.shard_of <= 1 and not args.no_extras
    int8_peak = None
    if (is_s8 or (default_run and world == 1)) and not args.no_extras:
        int8_peak = measure_int8_peak(ctx)
    int8_den = (int8_peak or {}).get("torch_int_mm") or 2.0 * peaks["bf16"]

    def frac_of_peak(tflops_per_gpu, s8):
        return tflops_per_gpu / (int8_den if s8 else peaks["bf16"])

    all_configs = None
    if default_run and world == 1:
        all_configs = {}
        for name in OTHER_CONFIGS:
            w = Workload(ctx, name, host_x=False)
            steps = 20
            v, ms = w.timed(steps, 3)
            u = w.unfused(steps, v)
            s8 = WORKLOADS[name][0][4] == "s8"
            all_configs[name] = {"value": v, "unit": "TOP/s" if s8 else "TFLOP/s", "ms_per_step": ms,
                                 "frac": frac_of_peak(v, s8), "unfused": u["value"],
                                 "fused_speedup": u["fused_speedup"], "kernels": w.kernels(), "steps": steps}
            del w, u
            torch.cuda.empty_cache()
    pipeline = None
    if default_run and world > 1:
        pipeline = {"workload": DESCR["pipeline"], "gather_check": gather_check(ctx)}
        for mode in ("fused", "nccl"):
            w = Workload(ctx, "pipeline", gather=mode, host_x=False)
            v, ms = w.timed(10, 3)
            gathered_bytes = 8192 * (57344 // 2) * 2             # the gate/up output, bf16
            pipeline[mode] = {"value": v, "unit": "TFLOP/s", "ms_per_step": ms,
                              "frac_per_gpu": frac_of_peak(v / world, False), "kernels": w.kernels(),
                              "nvlink_bytes_out_per_rank_per_step": gathered_bytes // world * (world - 1)}
            del w
            torch.cuda.empty_cache()
    clocks = sampler.stop(load_window=load_window)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak = int8_den if is_s8 else peaks["bf16"]
    achieved = flops_rank / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": None,
                "peak_source": ((f"int8 rate of torch._int_mm (cuBLASLt) at 8192^3 measured in this run; "
                                 f"this library's bare int8 kernel on the same problem: "
                                 f"{(int8_peak or {}).get('own_bare_kernel')}"
                                 if (int8_peak or {}).get("torch_int_mm") else
                                 "2 x measured bf16 burst (no int8 library GEMM could be timed)")
                                if is_s8 else f"bf16 burst, {peaks['src']}"),
                "frac_of_nominal": achieved / (4500.0 if is_s8 else 2250.0),
                "kernel": ",".join(sorted(set(kernels)))}
    if world == 1 and args.shard_of <= 1:
        roofline["traffic"] = load_traffic().get(args.workload)

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        v, rows, t, cores, cols = cpu_sample(stages, args.cpu_seconds, seed=0)
        cpu_baseline = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                        "sample": f"{rows} rows x {cols} columns x full K of the workload, {t:.1f} s of CPU time",
                        "library_gemm": cpu_library_gemm(stages)}

    sus_den = peaks.get("bf16_sustained")
    value_sustained = {
        "value": v_sus, "unit": "TFLOP/s", "ms_per_step": ms_sus, "steps": n_sus, "sm_mhz_median": sm_sus,
        "ms_x_mhz": (ms_sus * sm_sus) if sm_sus else None,
        "frac_of_sustained_peak": (v_sus / world / (sus_den * (2.0 if is_s8 else 1.0))) if sus_den else None,
        "how": "the timed step back to back for ~0.5 s (power-capped clocks); fraction of the measured "
               "bf16_tflops_sustained (x2 for int8); ms_x_mhz lets runs at different clocks be compared"}
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
                                   if world > 1 and has_chain else "")),
                   "l2": l2_note, "kernels": kernels},
        "value_sustained": value_sustained,
        "step_times": step_times,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "unfused": unfused,
        "gpu_launches": args.steps * n_stage, "clocks": clocks,
    }
    if int8_peak is not None:
        line["int8_peak"] = int8_peak
    if all_configs is not None:
        line["all_configs"] = all_configs
    if pipeline is not None:
        line["pipeline"] = pipeline
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
