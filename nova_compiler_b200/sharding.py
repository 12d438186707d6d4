"""Partitioning of the contraction across the GPUs of one box (one process per GPU, torch.distributed).

The reference has no multi-device code at all (its `#nova.device` attribute only separates host from
GPU); this is the plumbing the north star adds on top of the single-GPU kernels:

  * batched contractions (linalg.batch_matmul) shard by BATCH INDEX: rank r owns a contiguous range of
    batches; no rank needs another rank's data, so there is no collective on the data path;
  * one large GEMM shards by N-COLUMN SLABS: every rank holds A and its own column slab of B and produces
    the same column slab of C (bit-identical to those columns of the unsharded product); a collective is
    needed only when the caller wants the whole C on every rank: `gather_slabs` all-gathers the slabs
    (NCCL over NVLink on GPUs, gloo on CPU) and re-interleaves them into a row-major [M, N] matrix.

The contraction itself is passed in as a callable (default: ops.matmul, i.e. the CUDA kernels) so the
partitioning logic can be exercised on CPU ranks with another callable.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def batch_range(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """(first batch, number of batches) owned by `rank`: contiguous, sizes differ by at most one,
    every batch owned exactly once; ranks beyond `batch` own nothing."""
    if batch < 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("bad partition request")
    base, extra = divmod(batch, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def column_slab(n: int, world: int, rank: int, align: int = 64) -> Tuple[int, int]:
    """(first column, number of columns) of rank's slab.  Slab boundaries are multiples of `align`
    columns (64 columns = one 128-byte row of 16-bit elements, so every slab base keeps the 16-byte
    alignment the tensor maps need); the last non-empty slab takes the ragged remainder."""
    if n < 0 or world <= 0 or not 0 <= rank < world or align <= 0:
        raise ValueError("bad partition request")
    units = (n + align - 1) // align
    ustart, ucount = batch_range(units, world, rank)
    start = min(ustart * align, n)
    stop = min((ustart + ucount) * align, n)
    return start, stop - start


def sharded_batch_matmul(a: torch.Tensor, b: torch.Tensor, rank: int, world: int,
                         matmul_fn: Optional[Callable] = None) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """Computes this rank's batches of C = A @ B for A [B,M,K], B [B,K,N] (or [K,N] shared).
    Returns (C[start:start+count], (start, count)).  No communication."""
    if matmul_fn is None:
        from . import ops
        matmul_fn = ops.matmul
    start, count = batch_range(a.shape[0], world, rank)
    a_s = a[start:start + count]
    b_s = b if b.dim() == 2 else b[start:start + count]
    if count == 0:
        return a.new_empty((0, a.shape[1], b.shape[-1])), (start, 0)
    return matmul_fn(a_s, b_s), (start, count)


def slab_matmul(a: torch.Tensor, b: torch.Tensor, rank: int, world: int,
                matmul_fn: Optional[Callable] = None, **kw) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """Computes this rank's column slab of C = A @ B for A [M,K] (replicated) and B [K,N].  The slab of B
    is a strided view (row pitch stays N), not a copy.  Returns (C[:, start:start+count], (start, count))."""
    if matmul_fn is None:
        from . import ops
        matmul_fn = ops.matmul
    start, count = column_slab(b.shape[1], world, rank)
    if count == 0:
        return a.new_empty((a.shape[0], 0)), (start, 0)
    return matmul_fn(a, b[:, start:start + count], **kw), (start, count)


def gather_slabs(c_slab: torch.Tensor, n: int, group=None, out: Optional[torch.Tensor] = None,
                 align: int = 64) -> torch.Tensor:
    """All-gathers the ranks' column slabs into the full row-major [M, N] matrix on every rank.

    Transport: ONE all-gather (NCCL over NVLink on GPUs, gloo on CPU) into a [world, M, widest] staging buffer;
    slabs narrower than the widest (ragged N) are padded for the collective.  On GPUs the staging is then
    re-interleaved into [M, N] by one kernel of the library (nova_b200_interleave_slabs); CPU ranks, which only
    exercise the partition logic, copy the column blocks with torch.  `out` reuses a previous result's storage."""
    world = dist.get_world_size(group)
    m = c_slab.shape[0]
    widths = [column_slab(n, world, r, align)[1] for r in range(world)]
    wmax = max(widths) if widths else 0
    send = c_slab
    if c_slab.shape[1] != wmax or not c_slab.is_contiguous():
        send = c_slab.new_zeros((m, wmax))
        send[:, :c_slab.shape[1]] = c_slab
    staging = c_slab.new_empty((world, m, wmax))
    if c_slab.is_cuda:
        dist.all_gather_into_tensor(staging, send, group=group)
    else:
        dist.all_gather(list(staging.unbind(0)), send, group=group)
    if out is None:
        out = c_slab.new_empty((m, n))
    if c_slab.is_cuda:
        from . import _lib as L
        with torch.cuda.device(c_slab.device):
            L.check(L.load().nova_b200_interleave_slabs(staging.data_ptr(), out.data_ptr(), m, n, world, wmax, align,
                                                        c_slab.element_size(),
                                                        torch.cuda.current_stream().cuda_stream))
        staging.record_stream(torch.cuda.current_stream())
        return out
    for r in range(world):
        start, count = column_slab(n, world, r, align)
        if count:
            out[:, start:start + count] = staging[r][:, :count]
    return out


class PeerMatrix:
    """A row-major [rows, cols] matrix on every rank that the other ranks of the box can store into: the landing
    place of a slab-partitioned GEMM whose epilogue pushes its columns to all GPUs (nova_b200_gemm_push).

    Each rank allocates its matrix through the library (plain device memory with a CUDA IPC handle), the 64-byte
    handles travel through the process group, and every rank opens the others' matrices in its own address space.
    `local` is this rank's matrix as a torch tensor; `peer_ptrs` are the other ranks' base addresses as seen from here.
    One process per GPU on one machine."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, group=None):
        import ctypes as C
        from . import _lib as L
        self._L, self._lib = L, L.load()
        self.rows, self.cols, self.dtype, self.group = rows, cols, dtype, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        es = torch.empty((), dtype=dtype).element_size()
        self.nbytes = rows * cols * es
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        L.check(self._lib.nova_b200_peer_buffer_alloc(self.nbytes, C.byref(ptr), handle))
        self.ptr = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.peer_ptrs, self._opened = {}, []
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            p = C.c_void_p()
            L.check(self._lib.nova_b200_peer_buffer_open(h, C.byref(p)))
            self.peer_ptrs[r] = p.value
            self._opened.append(p.value)

        class _Raw:  # an integer view of the allocation; reinterpreted as `dtype` below
            __cuda_array_interface__ = {"shape": (rows, cols), "typestr": {1: "|u1", 2: "<i2", 4: "<i4"}[es],
                                        "data": (self.ptr, False), "version": 2}
        self._raw = _Raw()
        self.local = torch.as_tensor(self._raw, device=torch.device("cuda", torch.cuda.current_device())).view(dtype)

    def close(self):
        """Every rank stops using the peers' matrices, then the owners free them."""
        if getattr(self, "ptr", None) is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self._opened:
            self._lib.nova_b200_peer_buffer_close(p)
        dist.barrier(group=self.group)
        self.local = None
        self._lib.nova_b200_peer_buffer_free(self.ptr)
        self.ptr = None


def slab_matmul_push(a: torch.Tensor, b: torch.Tensor, out: "PeerMatrix", *, bias: Optional[torch.Tensor] = None,
                     act: Optional[str] = None) -> Tuple[int, int]:
    """This rank's column slab of C = act(A @ B + bias), written by the contraction's epilogue into `out.local` AND
    into every peer's matrix (plain stores over NVLink, overlapped with the contraction).  The whole C is valid on
    every rank once all ranks have passed a collective enqueued after this call (e.g. `dist.barrier()`).
    Returns this rank's (first column, width)."""
    import ctypes as C
    from . import _lib as L, ops
    rank, world = out.rank, out.world
    start, count = column_slab(b.shape[1], world, rank)
    if count == 0:
        return start, 0
    n = b.shape[1]
    es = out.local.element_size()
    bias_slab = bias[start:start + count].contiguous() if bias is not None else None
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    g.dtype_ab, g.dtype_c = ops._dt(a), ops._DT[out.dtype]
    g.batch, g.M, g.N, g.K = 1, a.shape[0], count, a.shape[1]
    g.A, g.lda = a.data_ptr(), a.stride(0)
    g.B, g.ldb = b.data_ptr() + start * b.element_size(), b.stride(0)      # the slab of B is a view: pitch stays N
    g.C, g.ldc = out.ptr + start * es, n
    g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = a.shape[0] * a.stride(0), 0, a.shape[0] * n
    g.act = ops._ACT[act]
    if bias_slab is not None:
        g.init, g.bias = L.INIT_BIAS_ROW, bias_slab.data_ptr()
    peers = (C.c_void_p * max(len(out.peer_ptrs), 1))(*[p + start * es for _, p in sorted(out.peer_ptrs.items())])
    L.check(L.load().nova_b200_gemm_push(C.byref(g), peers, len(out.peer_ptrs), ops._stream()))
    return start, count
