"""Host-side logic of the multi-GPU partition: ranges, and the statistics protocol that makes
the AUTO / scaling decision global.  Runs as two gloo ranks on CPU; the per-rank device work
is played by the CPU oracle behind a stand-in for the handle."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from cumpsgemm_b200.sharded import ShardedGemm, batch_range, column_range  # noqa: E402


def test_batch_range_covers_everything_once():
    for batch in (1, 7, 64, 512, 513):
        for world in (1, 2, 3, 4, 8):
            spans = [batch_range(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert batch_range(512, 8, 3) == (192, 256)       # config 4: 64 batches per GPU
    assert batch_range(64, 8, 7) == (56, 64)          # config 5a: 8 per GPU
    with pytest.raises(ValueError):
        batch_range(4, 2, 2)


def test_column_range_alignment():
    assert column_range(65536, 8, 2) == (16384, 24576)     # config 5b
    for n in (1000, 65536, 300):
        for world in (1, 2, 4, 8):
            spans = [column_range(n, world, r, align=256) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0
                assert a1 % 256 == 0 or a1 == n


class FakeHandle:
    """Plays the staged-statistics part of the handle with the CPU oracle.  Slots hold the same
    four words the library exports: max exponent bits, total, underflow, mode."""

    def __init__(self, oracle, params=(0.0, 2.0 ** -15, 0.0)):
        self.orc = oracle
        self.params = params
        self.slots = {}
        self.next = 2

    def exp_stats_begin(self):
        sid = self.next
        self.next += 1
        self.slots[sid] = {"max": 0.0, "total": 0, "uf": 0, "mode": 0}
        return sid

    def exp_stats_stage(self, stage, sid, m, n, ptr, ld, batch_size=1, stride=0, complex=None):
        x = ptr.numpy()
        s = self.slots[sid]
        ig, uf, _ = self.params
        if stage == 1:
            # tolerance 2: decision 1 inside the oracle never resets the raw counts
            r = self.orc.exp_stats(x, m, n, ld, batch_size, stride, ig, uf, 2.0)
            s.update(max=r["max_exp"], total=r["total"], uf=r["underflow"])
        elif stage == 2:
            if s["mode"] != 10:
                return
            r = self.orc.exp_stats(x, m, n, ld, batch_size, stride, (ig / 2) * s["max"],
                                   (uf / 2) * s["max"], 2.0)
            s.update(total=s["total"] + r["total"], uf=s["uf"] + r["underflow"])
        else:
            s["max"] = self.orc.exp_max(x, m, n, ld, batch_size, stride)

    def exp_stats_decide(self, decision, sid):
        s = self.slots[sid]
        tol = np.float32(self.params[2])
        if decision == 1:
            if (np.float32(s["uf"]) > np.float32(s["total"]) * tol) or (s["max"] > 0 and s["total"] == 0):
                s.update(mode=10, total=0, uf=0)
            else:
                s["mode"] = 1
        elif s["mode"] == 10:
            s["mode"] = 11 if np.float32(s["uf"]) <= np.float32(s["total"]) * tol else 2

    def exp_stats_export(self, sid, words):
        s = self.slots[sid]
        bits = int(np.float32(s["max"]).view(np.uint32))
        words.copy_(torch.tensor([bits, s["total"], s["uf"], s["mode"]], dtype=torch.int64))

    def exp_stats_import(self, sid, words):
        w = words.tolist()
        self.slots[sid].update(max=float(np.uint32(w[0]).view(np.float32)), total=w[1], uf=w[2],
                               mode=w[3])


def _worker(rank, world, port, case, out_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc

    batch, m, n = 6, 40, 30
    full = case_matrix(orc, case, batch * m * n)
    b0, b1 = batch_range(batch, world, rank)
    local = torch.from_numpy(full[b0 * m * n:b1 * m * n].copy())
    sg = ShardedGemm(FakeHandle(orc))
    sid = sg.global_exp_stats(m, n, local, m, b1 - b0, m * n)
    got = dict(sg.handle.slots[sid])
    mid = sg.global_exp_max(m, n, local, m, b1 - b0, m * n)
    got["max_only"] = sg.handle.slots[mid]["max"]
    out_queue.put((rank, got))
    dist.barrier()
    dist.destroy_process_group()


def case_matrix(orc, case, count):
    if case == "well":
        return orc.gen_uniform(1, count) + np.float32(2.0)
    if case == "tiny_rank1":       # rank 1's half is tiny: only the global view sees the range
        x = orc.gen_uniform(1, count) + np.float32(2.0)
        x[count // 2:] *= np.float32(2.0 ** -20)
        return x.astype(np.float32)
    if case == "all_tiny":
        return ((orc.gen_uniform(1, count) + np.float32(2.0)) * np.float32(2.0 ** -22)).astype(np.float32)
    raise ValueError(case)


@pytest.mark.parametrize("case", ["well", "tiny_rank1", "all_tiny"])
def test_global_statistics_equal_single_process(case, oracle):
    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    batch, m, n = 6, 40, 30
    full = case_matrix(oracle, case, batch * m * n)
    want = oracle.exp_stats(full, m, n, m, batch, m * n)
    for r in range(world):
        got = results[r]
        assert got["max"] == want["max_exp"] and got["mode"] == want["mode"]
        assert got["total"] == want["total"] and got["uf"] == want["underflow"]
        assert got["max_only"] == oracle.exp_max(full, m, n, m, batch, m * n)
    assert results[0] == results[1]
