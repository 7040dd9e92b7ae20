"""Two-GPU runs of the partitioned GEMM (one process per GPU, NCCL): batch ranges and C column
blocks, with the AUTO / FP16TCEC_SCALING decisions made global by the statistics all-reduce.
Skipped on boxes with a single GPU."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
N, T = 0, 1
FP16TCEC, TF32TCEC, AUTO, SCALING = 1, 2, 9, 11


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist

    from cumpsgemm_b200 import api
    from cumpsgemm_b200.sharded import ShardedGemm, batch_range, column_range
    from oracle import oracle as orc

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    h = api.Handle()
    h.use_current_torch_stream()
    sg = ShardedGemm(h)
    results = {}

    # ---- batch partition, AUTO: rank 1's batches of A are tiny, so only the global
    #      statistics see the whole exponent range of A
    batch, m, n, k = 6, 96, 160, 200
    a = (orc.gen_uniform(1, batch * m * k) + np.float32(2.0)).astype(np.float32)
    a[batch // 2 * m * k:] *= np.float32(2.0 ** -20)
    b = orc.gen_uniform(2, batch * k * n) + np.float32(2.0)
    b0, b1 = batch_range(batch, world, rank)
    nb = b1 - b0
    da = torch.from_numpy(a[b0 * m * k:b1 * m * k].copy()).cuda()
    db = torch.from_numpy(b[b0 * k * n:b1 * k * n].copy()).cuda()
    dc = torch.zeros(nb * m * n, device="cuda")
    for mode, key in ((AUTO, "auto"), (SCALING, "scaling")):
        dc.zero_()
        sg.gemm_strided_batch_local(N, N, m, n, k, 1.0, da, m, m * k, db, k, k * n, 0.0, dc, m,
                                    m * n, nb, mode)
        results[f"batch_{key}"] = dc.cpu().numpy().copy()
    # what a single GPU holding every batch decides
    ia = sg.global_exp_stats(m, k, da, m, nb, m * k)
    results["stats_a"] = np.array([h.get_max_exp(ia), *h.get_exp_stats(ia),
                                   int(h.get_exp_stats_compute_mode_level(ia))], dtype=np.float64)

    # ---- column partition: A lives on rank 0 only and is broadcast inside the call
    m2, n2, k2 = 200, 512, 300
    a2 = (orc.gen_uniform(3, m2 * k2) * np.float32(2.0 ** -22)).astype(np.float32)
    b2 = orc.gen_uniform(4, k2 * n2)
    c2 = orc.gen_uniform(5, m2 * n2)
    j0, j1 = column_range(n2, world, rank, align=128)
    dA = torch.from_numpy(a2.copy()).cuda() if rank == 0 else torch.zeros(m2 * k2, device="cuda")
    dB = torch.from_numpy(b2[j0 * k2:j1 * k2].copy()).cuda()
    dC = torch.from_numpy(c2[j0 * m2:j1 * m2].copy()).cuda()
    sg.gemm_column_block(N, N, m2, j1 - j0, k2, 1.0, dA, m2, dB, k2, 0.5, dC, m2, SCALING, root=0)
    results["col_scaling"] = dC.cpu().numpy().copy()
    results["col_range"] = np.array([j0, j1])
    assert h.kernel_status() == 0
    torch.cuda.synchronize()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    dist.destroy_process_group()
    h.destroy()


def test_two_gpu_partitions(oracle, tmp_path):
    import torch
    import torch.multiprocessing as mp

    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from cumpsgemm_b200.sharded import batch_range

    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    res = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]

    batch, m, n, k = 6, 96, 160, 200
    a = (oracle.gen_uniform(1, batch * m * k) + np.float32(2.0)).astype(np.float32)
    a[batch // 2 * m * k:] *= np.float32(2.0 ** -20)
    b = oracle.gen_uniform(2, batch * k * n) + np.float32(2.0)
    want = oracle.exp_stats(a, m, k, m, batch, m * k)
    for r in range(world):
        got = res[r]["stats_a"]
        assert (got[0], int(got[1]), int(got[2]), int(got[3])) == \
            (want["max_exp"], want["underflow"], want["total"], want["mode"])
    assert want["mode"] == TF32TCEC          # the range 2^-20 is visible only globally
    thr = oracle.error_threshold(True, k)
    for r in range(world):
        b0, b1 = batch_range(batch, world, r)
        for key in ("auto", "scaling"):
            out = res[r][f"batch_{key}"]
            for i in range(b0, b1):
                truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a[i * m * k:], m, b[i * k * n:], k, 0.0,
                                        None, m)
                assert oracle.residual(truth, out[(i - b0) * m * n:(i - b0 + 1) * m * n], m) < thr, \
                    (key, r, i)
    m2, n2, k2 = 200, 512, 300
    a2 = (oracle.gen_uniform(3, m2 * k2) * np.float32(2.0 ** -22)).astype(np.float32)
    b2 = oracle.gen_uniform(4, k2 * n2)
    c2 = oracle.gen_uniform(5, m2 * n2)
    truth = oracle.gemm_f64(N, N, m2, n2, k2, 1.0, a2, m2, b2, k2, 0.5, c2, m2)
    full = np.concatenate([res[r]["col_scaling"] for r in range(world)])
    assert [tuple(res[r]["col_range"]) for r in range(world)] == [(0, 256), (256, 512)]
    assert oracle.residual(truth, full, m2) < oracle.error_threshold(True, k2)
