"""Multi-GPU host logic on CPU: column sharding, the all-gather of output shards (gloo,
world_size 2) and the K-slab view the consumer stage reads the gathered buffer through."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_columns(xf):
    sh = xf.sharding
    assert sh.shard_columns(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert sh.shard_columns(1024, 8, 7, multiple=128) == (896, 1024)      # one KV head per GPU
    assert sh.shard_columns(57344, 8, 0, multiple=sh.stage_multiple("k2", compact=True)) == (0, 7168)
    with pytest.raises(ValueError):
        sh.shard_columns(1000, 3, 0)          # uneven
    with pytest.raises(ValueError):
        sh.shard_columns(1024, 16, 0, multiple=128)   # half a head
    with pytest.raises(ValueError):
        sh.shard_columns(1024, 4, 4)
    cover = [sh.shard_columns(4096, 4, r, 128) for r in range(4)]
    assert cover[0][0] == 0 and cover[-1][1] == 4096 and all(a[1] == b[0] for a, b in zip(cover, cover[1:]))


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as o
    import xefuse_loader
    sh = xefuse_loader.load().sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # stage 1 (gate/up, k2 compact) sharded by columns; stage 2 (down) contracts over its output
        M, K1, N1, N2 = 24, 64, 1024 * world, 32
        rng = np.random.default_rng(7)                      # same stream on every rank: replicated X
        X = o.f32_to_bf16(rng.standard_normal((M, K1)).astype(np.float32))
        R = o.compute_rstd(X)
        W1 = o.f32_to_bf16((rng.standard_normal((K1, N1)) * K1 ** -0.5).astype(np.float32))
        W2 = o.f32_to_bf16((rng.standard_normal((N1 // 2, N2)) * (N1 // 2) ** -0.5).astype(np.float32))
        lo, hi = sh.shard_columns(N1, world, rank, sh.stage_multiple("k2", compact=True))
        d_shard = o.epilogue(o.gemm_bf16(X, W1[:, lo:hi]), row=R, pair="swiglu", compact=True)
        # gloo has no 16-bit integer type: move the bf16 bit patterns as bytes
        shard_t = torch.from_numpy(d_shard.view(np.uint8).copy())
        gathered_b = torch.empty(sh.gathered_shape(M, (hi - lo) // 2 * 2, world), dtype=torch.uint8)
        sh.all_gather_shards(dist, shard_t, gathered_b)
        gathered = gathered_b.view(torch.int16)
        # the slab view equals the unsharded stage output
        full = o.epilogue(o.gemm_bf16(X, W1), row=R, pair="swiglu", compact=True)
        same = np.array_equal(sh.slabs_to_matrix(gathered).numpy().view(np.uint16), full)
        # consumer over K slabs == consumer over the full matrix (what a_k_slab addressing does)
        slabs = gathered.numpy().view(np.uint16)
        ks = slabs.shape[2]
        acc = sum(o.gemm_bf16(slabs[g], W2[g * ks:(g + 1) * ks]) for g in range(world))
        ref = o.gemm_bf16(full, W2)
        close = bool(np.abs(acc - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()))
        # a rank with a mismatched buffer is refused on the host, before any collective
        try:
            sh.all_gather_shards(dist, shard_t, torch.empty((world, M, 3), dtype=torch.uint8))
            refused = False
        except ValueError:
            refused = True
        q.put((rank, same, close, refused))
    except Exception as e:  # report instead of leaving the parent waiting
        q.put((rank, False, False, repr(e)))
    finally:
        dist.destroy_process_group()


def test_all_gather_of_column_shards_gloo_world2(xf, oracle):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in res), res


@pytest.mark.gpu
def test_consumer_reads_gathered_k_slabs_on_gpu(capi, oracle, cuda):
    """A stored as G K-slabs (the gathered layout) gives the same result as the plain [M,K] matrix."""
    import torch
    import parity_cases as pc
    from conftest import bf16_bits
    G, M, Ks, N = 4, 256, 512, 384
    rng = np.random.default_rng(3)
    A = oracle.f32_to_bf16(rng.standard_normal((M, G * Ks)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.standard_normal((G * Ks, N)) * (G * Ks) ** -0.5).astype(np.float32))
    gamma = rng.normal(1, 0.02, N).astype(np.float32)
    res = oracle.f32_to_bf16(rng.standard_normal((M, N)).astype(np.float32))
    slabs = np.ascontiguousarray(A.reshape(M, G, Ks).transpose(1, 0, 2))       # [G][M, Ks]
    t = lambda a, bf=True: (torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16) if bf
                            else torch.from_numpy(a)).to(cuda)
    for flags in (0, capi.FLAG_FORCE_1CTA | capi.FLAG_FORCE_BN128 | capi.FLAG_FORCE_KS1):
        D = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda)
        plan = capi.GemmPlan(t(slabs), t(B), D, residual=t(res), col_scale=t(gamma, False), a_k_slabs=True, flags=flags)
        plan.run()
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        want = oracle.epilogue(oracle.gemm_bf16(A, B), residual=res, col=gamma)
        assert pc.compare_bf16(oracle, bf16_bits(D), want)[0] == 0, plan.kernel_name


@pytest.mark.gpu
def test_output_copies_from_the_epilogue_on_gpu(capi, oracle, cuda):
    """xf_gemm_desc.D_peer: every output tile is also stored to the extra destinations (here local
    buffers standing in for the peers' gathered slabs), for TMA and for plain stores."""
    import torch
    import parity_cases as pc
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, "k2_compact", 392, 640, 200, 13)
    _, want = pc.expected(oracle, "k2_compact", d)
    t = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(cuda)
    A, B, R = t(d["A"]), t(d["B"]), torch.from_numpy(d["scale"]).to(cuda)
    for flags in (0, capi.FLAG_DIRECT_STORE):
        D = torch.zeros((392, 320), dtype=torch.bfloat16, device=cuda)
        copies = [torch.zeros_like(D) for _ in range(3)]
        plan = capi.GemmPlan(A, B, D, row_scale=R, pair="swiglu", compact=True, flags=flags,
                             d_peer_ptrs=[c.data_ptr() for c in copies])
        plan.run()
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        assert pc.compare_bf16(oracle, bf16_bits(D), want)[0] == 0
        for c in copies:
            assert torch.equal(c.view(torch.int16), D.view(torch.int16))


@pytest.mark.gpu
def test_sharded_stages_with_fused_and_nccl_gather_on_2_gpus(capi, oracle, cuda):
    """Needs two GPUs on the box: producer shards -> gathered K slabs (peer stores from the
    epilogue, and ncclAllGather) -> consumer, every rank checked against the oracle."""
    import subprocess
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible: the 2-rank check needs two")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
                        os.path.join(ROOT, "tests", "multi_gpu_check.py")],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "MULTI_GPU_CHECK PASSED" in r.stdout, r.stdout[-3000:]
