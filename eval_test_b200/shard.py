"""Sharding the four problems over the GPUs of one box: one process per GPU, no K split, so no reduction and
no collective on the data path.

* GEMM / dual GEMM: rank r owns columns ``[r*N/g, (r+1)*N/g)`` of C, i.e. rows of B (B1, B2) and of their scales;
  A and its scales are replicated.  Because the swizzled scale layout is ``[rows/128][K/64][512 B]``, a row range
  aligned to 128 is a contiguous byte range of the scale buffer.
* GEMV: rank r owns rows ``[r*M/g, (r+1)*M/g)`` of A, of its scales and of the output; the vector is replicated.
* grouped GEMM: whole groups are assigned to ranks, balanced by weight bytes (the layer is HBM-bound on weights).

The shards are materialised once, at set-up (weights are static); every shard is again a valid input tuple of the
corresponding ``custom_kernel``.  ``gather_*`` reassemble the full output with an all-gather (NCCL over NVLink on
GPUs, gloo on CPU); it is optional and never part of a timed kernel.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import formats as F


def _check_even(total: int, world: int, what: str) -> int:
    if total % (128 * world) != 0:
        raise ValueError(f"{what} = {total} must be a multiple of 128 * world_size ({128 * world})")
    return total // world


def _rows(t: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Rows [lo, hi) of a ``[rows, cols, L]`` batch-last tensor, re-laid out batch-outermost."""
    return F.batch_last(t[lo:hi].permute(2, 0, 1).contiguous())


def _scale_rows(p: torch.Tensor, lo: int, hi: int, K: int) -> torch.Tensor:
    """128-row blocks [lo/128, hi/128) of a 6-D swizzled scale view, as a fresh view over its own buffer."""
    L = p.shape[5]
    blk = p[:, :, lo // 128: hi // 128].permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).reshape(-1)
    return F.permuted_view(blk, hi - lo, K, L)


def shard_gemm(data, rank: int, world: int):
    """Column shard of a GEMM input tuple ``(a, b, sfa, sfb, sfa_p, sfb_p, c)``."""
    a, b, sfa, sfb, sfa_p, sfb_p, c = data
    n, k = b.shape[0], 2 * b.shape[1]
    step = _check_even(n, world, "N")
    lo, hi = rank * step, (rank + 1) * step
    c_loc = F.batch_last(torch.empty((c.shape[2], c.shape[0], step), dtype=c.dtype, device=c.device))
    return (a, _rows(b, lo, hi), sfa, _rows(sfb, lo, hi), sfa_p, _scale_rows(sfb_p, lo, hi, k), c_loc)


def shard_dual_gemm(data, rank: int, world: int):
    a, b1, b2, sfa, sfb1, sfb2, sfa_p, sfb1_p, sfb2_p, c = data
    n, k = b1.shape[0], 2 * b1.shape[1]
    step = _check_even(n, world, "N")
    lo, hi = rank * step, (rank + 1) * step
    c_loc = F.batch_last(torch.empty((c.shape[2], c.shape[0], step), dtype=c.dtype, device=c.device))
    return (a, _rows(b1, lo, hi), _rows(b2, lo, hi), sfa, _rows(sfb1, lo, hi), _rows(sfb2, lo, hi), sfa_p,
            _scale_rows(sfb1_p, lo, hi, k), _scale_rows(sfb2_p, lo, hi, k), c_loc)


def shard_gemv(data, rank: int, world: int):
    """Row shard of a GEMV input tuple (``b`` is the 128-row padded vector, replicated)."""
    a, b, sfa, sfb, sfa_p, sfb_p, c = data
    m, k = a.shape[0], 2 * a.shape[1]
    step = _check_even(m, world, "M")
    lo, hi = rank * step, (rank + 1) * step
    c_loc = F.batch_last(torch.empty((c.shape[2], step, 1), dtype=c.dtype, device=c.device))
    return (_rows(a, lo, hi), b, _rows(sfa, lo, hi), sfb, _scale_rows(sfa_p, lo, hi, k), sfb_p, c_loc)


def assign_groups(ms: list[int], world: int) -> list[list[int]]:
    """Group indices per rank: non-empty groups first, largest M first, each to the rank with the fewest groups
    (weight bytes), ties to the smaller sum of M; empty groups are dealt last (they cost nothing)."""
    ranks: list[list[int]] = [[] for _ in range(world)]
    load = [(0, 0)] * world  # (non-empty groups, sum M)
    order = sorted(range(len(ms)), key=lambda i: (ms[i] == 0, -ms[i], i))
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        ranks[r].append(i)
        if ms[i] > 0:
            load[r] = (load[r][0] + 1, load[r][1] + ms[i])
    return [sorted(r) for r in ranks]


def shard_grouped_gemm(data, rank: int, world: int):
    """The groups of ``rank`` (tuple of sub-lists) and their indices in the full problem."""
    abc, sfs, sfs_p, sizes = data
    mine = assign_groups([s[0] for s in sizes], world)[rank]
    pick = lambda xs: [xs[i] for i in mine]
    return (pick(abc), pick(sfs), pick(sfs_p), pick(sizes)), mine


def gather_cols(c_local: torch.Tensor, world: int) -> torch.Tensor:
    """All-gather of column shards ``[M, N/g, L]`` into the full ``[M, N, L]`` (optional; not on the timed path)."""
    if world == 1:
        return c_local
    flat = c_local.permute(2, 0, 1).contiguous()              # [L, M, N/g]
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat)
    return F.batch_last(torch.cat(parts, dim=2).contiguous())


def gather_rows(c_local: torch.Tensor, world: int) -> torch.Tensor:
    """All-gather of GEMV row shards ``[M/g, 1, L]`` into ``[M, 1, L]``."""
    if world == 1:
        return c_local
    flat = c_local.permute(2, 0, 1).contiguous()              # [L, M/g, 1]
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat)
    return F.batch_last(torch.cat(parts, dim=1).contiguous())


# ----------------------------------------------------------------------------------------------- fused all-gather
class GatheredOutput:
    """The full ``[M, N, L]`` fp16 output of an N-sharded GEMM, one copy per rank, that every rank's kernel writes its
    column slice into directly (``nvfp4_gemm_allgather``): a symmetric-memory buffer whose copies on the other ranks
    are mapped into this process.  ``ptrs`` may also be given explicitly (buffers of one device: single-GPU tests)."""

    def __init__(self, m: int, n: int, l: int, device, group=None, ptrs=None, buf=None):
        self.m, self.n, self.l = m, n, l
        if ptrs is not None:
            self.buf, self.ptrs, self.group = buf, list(ptrs), None
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self.group = group if group is not None else dist.group.WORLD
            self.buf = symm_mem.empty((l, m, n), dtype=torch.float16, device=device)
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            # the handle lists each rank's symmetric buffer; this tensor may start at an offset inside it
            base = [int(p) for p in self.handle.buffer_ptrs]
            off = self.buf.data_ptr() - base[self.handle.rank]
            self.ptrs = [p + off for p in base]
        self.world = len(self.ptrs)

    def view(self) -> torch.Tensor:
        """The local copy as ``[M, N, L]`` (the layout of the reference's ``c``)."""
        return F.batch_last(self.buf)

    def _stream_barrier(self):
        if self.group is not None and self.world > 1:
            if getattr(self, "_flag", None) is None:
                self._flag = torch.zeros(1, dtype=torch.float32, device=self.buf.device)
            dist.all_reduce(self._flag, group=self.group)

    def wait_all(self):
        """Stream-ordered: what follows on the current stream runs after every rank's kernel has finished, so every
        copy is complete.  (A one-element all-reduce: unlike ``dist.barrier`` it does not block the host.)"""
        self._stream_barrier()

    def release(self):
        """Stream-ordered, the other half of the protocol: call it after the consumers of this rank's copy have
        been enqueued and before the next ``gemm_allgather`` into the same buffer.  What follows on the current
        stream runs only after every rank has got that far, so no rank's next launch overwrites a copy that a peer
        is still reading.  ``wait_all`` alone only protects against reading too early.  (Alternating between two
        ``GatheredOutput`` buffers does the same job without the second barrier.)"""
        self._stream_barrier()


def _ptr_array(ptrs):
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def gemm_allgather(shard, out: GatheredOutput, rank: int, alpha: float = 1.0):
    """``shard``: this rank's tuple from ``shard_gemm`` (its ``c`` is not used).  Writes the rank's columns into every
    rank's copy of ``out``; call ``out.wait_all()`` before reading, and ``out.release()`` after the readers and before
    the next launch into the same ``out``."""
    from . import _args, _lib
    a, b, _, _, sfa_p, sfb_p, _ = shard
    m, k2, l = a.shape
    n_loc, k = b.shape[0], 2 * k2
    if (m, n_loc * out.world, l) != (out.m, out.n, out.l):
        raise ValueError(f"gemm_allgather: shard {m} x {n_loc} x {l} does not tile an output {out.m} x {out.n} x {out.l} "
                         f"over {out.world} ranks")
    with torch.cuda.device(a.device):
        code = _lib.load().nvfp4_gemm_allgather(
            _args.operand_ptr(a, m, k2, l, "a"), _args.operand_ptr(b, n_loc, k2, l, "b"),
            _args.scales_ptr(sfa_p, m, k, l, "sfa_permuted"), _args.scales_ptr(sfb_p, n_loc, k, l, "sfb_permuted"),
            _ptr_array(out.ptrs), out.world, rank, m, n_loc, k, l, float(alpha), _args.stream_ptr(a.device))
    _lib.check(code, "nvfp4_gemm_allgather")
    return out


def dual_gemm_allgather(shard, out: GatheredOutput, rank: int, alpha: float = 1.0):
    from . import _args, _lib
    a, b1, b2, _, _, _, sfa_p, sfb1_p, sfb2_p, _ = shard
    m, k2, l = a.shape
    n_loc, k = b1.shape[0], 2 * k2
    if (m, n_loc * out.world, l) != (out.m, out.n, out.l):
        raise ValueError("dual_gemm_allgather: the shard does not tile the output")
    with torch.cuda.device(a.device):
        code = _lib.load().nvfp4_dual_gemm_allgather(
            _args.operand_ptr(a, m, k2, l, "a"), _args.operand_ptr(b1, n_loc, k2, l, "b1"),
            _args.operand_ptr(b2, n_loc, k2, l, "b2"), _args.scales_ptr(sfa_p, m, k, l, "sfa_permuted"),
            _args.scales_ptr(sfb1_p, n_loc, k, l, "sfb1_permuted"), _args.scales_ptr(sfb2_p, n_loc, k, l, "sfb2_permuted"),
            _ptr_array(out.ptrs), out.world, rank, m, n_loc, k, l, float(alpha), _args.stream_ptr(a.device))
    _lib.check(code, "nvfp4_dual_gemm_allgather")
    return out
