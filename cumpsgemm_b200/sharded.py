"""Multi-GPU partitioning of the TCEC GEMM path (one process per GPU).

The reference is single-GPU (device 0 is hard-coded, ``src/handle.cu:12-21``);
this module adds the two partitions the path admits without any collective in
the inner loop:

* strided-batch calls are split by contiguous batch ranges, every rank keeping
  its own A_b, B_b, C_b;
* a single large GEMM is split by column blocks of C: B and C blocks are
  resident on their rank, A is broadcast once over NCCL into each rank's own
  memory, after which every kernel reads local memory only.

For ``AUTO`` and ``FP16TCEC_SCALING`` the reference's decision and scale factor
cover the whole operand (``src/exp_stats.cu:81-82,163-165``), so the statistics
slots are combined over the ranks between the stages (max of the exponent bits, sums of
the two counters; one small all-gather per stage for both operands together); every rank
then takes the same decision as a 1-GPU run would.
"""
from __future__ import annotations

from typing import Tuple

from .api import CUBLAS_OP_N, ComputeMode, Handle


def batch_range(batch_count: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of the batches owned by `rank`; sizes differ by at most one."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world size")
    base, extra = divmod(batch_count, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def column_range(n: int, world_size: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous [begin, end) of the columns of C (and of op(B)) owned by `rank`.

    Block boundaries are multiples of `align` (except the end of the matrix)."""
    if world_size <= 0 or not (0 <= rank < world_size) or align <= 0:
        raise ValueError("bad rank / world size / alignment")
    blocks = (n + align - 1) // align
    b0, b1 = batch_range(blocks, world_size, rank)
    return min(b0 * align, n), min(b1 * align, n)


class ShardedGemm:
    """Runs one rank's share of a partitioned GEMM.  `group` is a torch.distributed group
    (None = default group); with a world size of 1 no collective is issued."""

    def __init__(self, handle: Handle, group=None):
        import torch
        import torch.distributed as dist

        self.handle = handle
        self.group = group
        self.dist = dist
        self.torch = torch
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    # ------------------------------------------------------------------ statistics
    def _global_rank(self, group_rank: int) -> int:
        if self.group is None:
            return group_rank
        return self.dist.get_global_rank(self.group, group_rank)

    def _export(self, sids, device):
        """[len(sids), 4] int64 on `device`: the exported words of the slots."""
        torch = self.torch
        w = torch.zeros(len(sids), 4, dtype=torch.int64, device=device)
        for i, sid in enumerate(sids):
            self.handle.exp_stats_export(sid, w[i])
        return w

    def _gather(self, w):
        """[world, ...] stack of every rank's `w` (one collective, whatever the slot count)."""
        torch, dist = self.torch, self.dist
        w = w.contiguous()
        out = torch.empty((self.world_size,) + tuple(w.shape), dtype=w.dtype, device=w.device)
        try:
            dist.all_gather_into_tensor(out, w, group=self.group)
        except (RuntimeError, NotImplementedError):   # a backend without the flat form
            parts = [torch.empty_like(w) for _ in range(self.world_size)]
            dist.all_gather(parts, w, group=self.group)
            out = torch.stack(parts)
        return out

    def _global_stats(self, operands, full: bool):
        """Statistics slots of several operands whose content equals what one GPU holding the
        whole operands would compute.  operands: (m, n, ptr, ld, batch_size, stride, replicated)
        with `replicated` = every rank holds the same full operand (no reduction needed).
        full = False: maximum exponent only (FP16TCEC_SCALING).  All operands share the
        collectives: one all-gather of the slot words per stage, reduced locally (max over ranks
        of word 0, the exponent bits; sum over ranks of words 1..2, the counters)."""
        h = self.handle
        sids = [h.exp_stats_begin() for _ in operands]
        for sid, o in zip(sids, operands):
            h.exp_stats_stage(1 if full else 3, sid, *o[:6])
        shared = [sid for sid, o in zip(sids, operands) if not o[6]] if self.world_size > 1 else []
        device = operands[0][2].device
        if shared:
            w = self._export(shared, device)
            g = self._gather(w)
            w[:, 0] = g[:, :, 0].amax(dim=0)
            if full:
                w[:, 1:3] = g[:, :, 1:3].sum(dim=0)
            for i, sid in enumerate(shared):
                h.exp_stats_import(sid, w[i])
        if not full:
            return sids
        for sid in sids:
            h.exp_stats_decide(1, sid)
        # After decision 1 the counters are either zero (undecided: stage 2 recounts) or already
        # global (decided: stage 2 is skipped on the device).  Only what stage 2 adds locally may
        # be summed over the ranks.
        base = self._export(shared, device) if shared else None
        for sid, o in zip(sids, operands):
            h.exp_stats_stage(2, sid, *o[:6])
        if shared:
            now = self._export(shared, device)
            delta = self._gather(now[:, 1:3] - base[:, 1:3]).sum(dim=0)
            now[:, 1:3] = base[:, 1:3] + delta
            for i, sid in enumerate(shared):
                h.exp_stats_import(sid, now[i])
        for sid in sids:
            h.exp_stats_decide(2, sid)
        return sids

    def global_exp_stats(self, m, n, ptr, ld, batch_size=1, stride=0, replicated=False) -> int:
        """Statistics slot (both stages and decisions) of one operand spread over the ranks."""
        return self._global_stats([(m, n, ptr, ld, batch_size, stride, replicated)], True)[0]

    def global_exp_max(self, m, n, ptr, ld, batch_size=1, stride=0, replicated=False) -> int:
        """Maximum-exponent slot of one operand spread over the ranks."""
        return self._global_stats([(m, n, ptr, ld, batch_size, stride, replicated)], False)[0]

    @staticmethod
    def _operand(op, rows, cols, ptr, ld, batch, stride, replicated):
        sm, sn = (rows, cols) if op == CUBLAS_OP_N else (cols, rows)
        return (sm, sn, ptr, ld, batch, stride if batch > 1 else 0, replicated)

    # ------------------------------------------------------------------ batch partition
    def gemm_strided_batch_local(self, op_A, op_B, m, n, k, alpha, A, lda, stridea, B, ldb,
                                 strideb, beta, Cmat, ldc, stridec, local_batch_count, mode):
        """This rank's batches of a strided-batch GEMM whose batches are spread over the ranks.
        A, B, Cmat hold only the local batches."""
        mode = ComputeMode(mode)
        h = self.handle
        if mode in (ComputeMode.AUTO, ComputeMode.FP16TCEC_SCALING):
            ida, idb = self._global_stats(
                [self._operand(op_A, m, k, A, lda, local_batch_count, stridea, False),
                 self._operand(op_B, k, n, B, ldb, local_batch_count, strideb, False)],
                mode == ComputeMode.AUTO)
            return h.gemm_strided_batch_with_stats(op_A, op_B, m, n, k, alpha, A, lda, stridea, B,
                                                   ldb, strideb, beta, Cmat, ldc, stridec,
                                                   local_batch_count, mode, ida, idb)
        return h.gemm_strided_batch(op_A, op_B, m, n, k, alpha, A, lda, stridea, B, ldb, strideb,
                                    beta, Cmat, ldc, stridec, local_batch_count, mode)

    # ------------------------------------------------------------------ column partition
    def gemm_column_block(self, op_A, op_B, m, n_local, k, alpha, A, lda, B_local, ldb, beta,
                          C_local, ldc, mode, root: int = 0, broadcast_A: bool = True):
        """This rank's column block C[:, J] = alpha*op(A)*op(B)[:, J] + beta*C[:, J].

        A must be a tensor of the full stored extent on every rank; its content is taken from
        `root` (one NCCL broadcast into local memory) unless broadcast_A is False, in which
        case every rank already holds it."""
        mode = ComputeMode(mode)
        h = self.handle
        if broadcast_A and self.world_size > 1:
            self.dist.broadcast(A, src=self._global_rank(root), group=self.group)
        if mode in (ComputeMode.AUTO, ComputeMode.FP16TCEC_SCALING):
            ida, idb = self._global_stats(
                [self._operand(op_A, m, k, A, lda, 1, 0, True),
                 self._operand(op_B, k, n_local, B_local, ldb, 1, 0, False)],
                mode == ComputeMode.AUTO)
            return h.gemm_strided_batch_with_stats(op_A, op_B, m, n_local, k, alpha, A, lda, 0,
                                                   B_local, ldb, 0, beta, C_local, ldc, 0, 1,
                                                   mode, ida, idb)
        return h.gemm(op_A, op_B, m, n_local, k, alpha, A, lda, B_local, ldb, beta, C_local, ldc,
                      mode)
