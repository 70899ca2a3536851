"""Run under torch.distributed.run with one rank per GPU (2..8 GPUs of one box):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 tests/multi_gpu_check.py

A gate/up stage (k2, compact) is column-sharded over the ranks; its output shards reach every
rank's gathered [G][M, Ns] buffer (a) by peer stores from the producer's epilogue and (b) by
ncclAllGather; a down-projection (k0a) then contracts over the gathered K slabs.  Every rank
checks both gathered buffers and its down-projection shard against the CPU oracle and rank 0
prints MULTI_GPU_CHECK PASSED.  Failures are reported on the host; no rank leaves mid-step.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import torch.distributed as dist
    import oracle as o
    import parity_cases as pc
    import xefuse_loader
    xf = xefuse_loader.load()
    capi, sh = xf.capi, xf.sharding
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    try:
        M, K1, N2 = 384, 320, 512
        N1 = 2 * 256 * 2 * world              # gate/up columns; each rank's compact shard is 512 wide
        rng = np.random.default_rng(11)        # identical on every rank: replicated inputs
        X = o.f32_to_bf16(rng.standard_normal((M, K1)).astype(np.float32))
        R = o.compute_rstd(X)
        W1 = o.f32_to_bf16((rng.standard_normal((K1, N1)) * K1 ** -0.5).astype(np.float32))
        W2 = o.f32_to_bf16((rng.standard_normal((N1 // 2, N2)) * (N1 // 2) ** -0.5).astype(np.float32))
        res = o.f32_to_bf16(rng.standard_normal((M, N2)).astype(np.float32))
        gamma = rng.normal(1, 0.02, N2).astype(np.float32)
        t = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(dev)
        bits = lambda x: x.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)

        lo, hi = sh.shard_columns(N1, world, rank, sh.stage_multiple("k2", compact=True))
        ns = (hi - lo) // 2
        tX, tR, tW1 = t(X), torch.from_numpy(R).to(dev), t(np.ascontiguousarray(W1[:, lo:hi]))
        full = o.epilogue(o.gemm_bf16(X, W1), row=R, pair="swiglu", compact=True)        # [M, N1/2]

        # (a) all-gather fused into the producer's epilogue
        gb = sh.GatherBuffer(dist, M, ns, torch.bfloat16, dev)
        gb.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        prod = capi.GemmPlan(tX, tW1, gb.local_shard, row_scale=tR, pair="swiglu", compact=True,
                             d_peer_ptrs=gb.peer_slab_ptrs())
        prod.run()
        gb.barrier()
        torch.cuda.synchronize()
        got = bits(sh.slabs_to_matrix(gb.tensor))
        ok &= pc.compare_bf16(o, got, full)[0] == 0 and prod.device_status() == 0

        # (b) separate ncclAllGather of the same shard
        shard = torch.zeros((M, ns), dtype=torch.bfloat16, device=dev)
        gathered = torch.zeros(sh.gathered_shape(M, ns, world), dtype=torch.bfloat16, device=dev)
        capi.GemmPlan(tX, tW1, shard, row_scale=tR, pair="swiglu", compact=True).run()
        sh.all_gather_shards(dist, shard, gathered)
        torch.cuda.synchronize()
        ok &= bool(torch.equal(gathered.view(torch.int16), gb.tensor.view(torch.int16)))

        # consumer: down projection over the gathered K slabs, N2 columns sharded again
        lo2, hi2 = sh.shard_columns(N2, world, rank, 2)
        D = torch.zeros((M, hi2 - lo2), dtype=torch.bfloat16, device=dev)
        cons = capi.GemmPlan(gb.tensor, t(np.ascontiguousarray(W2[:, lo2:hi2])), D,
                             residual=t(np.ascontiguousarray(res[:, lo2:hi2])),
                             col_scale=torch.from_numpy(gamma[lo2:hi2].copy()).to(dev), a_k_slabs=True)
        cons.run()
        torch.cuda.synchronize()
        want = o.epilogue(o.gemm_bf16(full, W2[:, lo2:hi2]), residual=res[:, lo2:hi2], col=gamma[lo2:hi2])
        ok &= pc.compare_bf16(o, bits(D), want)[0] == 0 and cons.device_status() == 0
    except Exception as e:   # report on the host, then join the final collective like everyone else
        print(f"rank {rank}: {e!r}", flush=True)
        ok = False
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("MULTI_GPU_CHECK PASSED" if int(flag.item()) == 1 else "MULTI_GPU_CHECK FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
