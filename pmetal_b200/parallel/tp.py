"""Tensor-parallel linear layers whose collective is fused into the GEMM kernel (csrc/tp_fused.cu).

* ``ColumnParallelLinear`` — sequence-sharded input, output features sharded: ``Y[M, N/w] = allgather(X) @ W_loc^T``.
  The kernel's TMA producer reads every rank's input shard straight from peer memory.
* ``RowParallelLinear`` — input features sharded, output rows scattered: ``Y_r = reduce_scatter(X_loc @ W_loc^T)``.
  The kernel's epilogue pushes partial tiles into the owner's staging buffer and each rank sums its own rows.

Both keep their exchange buffers in ``torch.distributed._symmetric_memory``; ``*_nccl`` are the library-collective
baselines the fused kernels are measured against. Weight sharding follows the reference's directives
(crates/pmetal-distributed/src/tensor_parallel/sharding.rs; forward semantics of sharded_linear.rs:41-106)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist


def _symm(numel: int, dtype, group):
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(numel, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
    h = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
    return t, h


class _FusedTpBase:
    def __init__(self, group=None, timeout_s: float = 10.0, max_ctas: int = 0):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.timeout_s, self.max_ctas = timeout_s, max_ctas
        self.pad, hpad = _symm(32, torch.int32, group)
        self.pad.zero_()
        self._arr = ctypes.c_ulonglong * self.world
        self._pads = self._arr(*[int(x) for x in hpad.buffer_ptrs])
        self._keep = [hpad]

    def _sync_setup(self):
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def _launch(self, mode, x_ptrs, ldx, w, out, stage_ptrs, M, N, K, gathered=None, blk_ready=None):
        from ..ops import native
        lib = native.lib()
        lib.pm_tp_gemm.restype = ctypes.c_int
        rc = lib.pm_tp_gemm(ctypes.c_int(mode), x_ptrs, ctypes.c_int(ldx), native._p(w), ctypes.c_int(w.stride(0)),
                            native._p(out), ctypes.c_int(out.stride(0)), stage_ptrs, self._pads, ctypes.c_int(self.rank),
                            ctypes.c_int(self.world), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                            native._p(gathered), native._p(blk_ready), ctypes.c_double(self.timeout_s), ctypes.c_int(self.max_ctas),
                            native._p(native.status_word()), native._stream())
        native._chk(rc, "pm_tp_gemm")


class ColumnParallelLinear(_FusedTpBase):
    """``weight``: this rank's [N_loc, K] slice (bf16). Inputs go through ``input_buffer`` ([M/world, K], symmetric)."""

    def __init__(self, weight: torch.Tensor, rows_per_rank: int, group=None, **kw):
        super().__init__(group, **kw)
        assert weight.dtype == torch.bfloat16 and weight.is_contiguous() and rows_per_rank % 128 == 0
        self.weight = weight
        self.rows = rows_per_rank
        self.K = weight.shape[1]
        x, hx = _symm(rows_per_rank * self.K, torch.bfloat16, group)
        self.input_buffer = x.view(rows_per_rank, self.K)
        self._x_ptrs = self._arr(*[int(p) for p in hx.buffer_ptrs])
        self._keep.append(hx)
        # remote shards are staged into this local buffer by the kernel's copy warps; one flag per 128-row block
        self.gathered = torch.empty(rows_per_rank * self.world, self.K, dtype=torch.bfloat16, device=weight.device)
        self.blk_ready = torch.zeros(rows_per_rank * self.world // 128, dtype=torch.int32, device=weight.device)
        self._sync_setup()

    def forward(self, x_local: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x_local is not None and x_local.data_ptr() != self.input_buffer.data_ptr():
            self.input_buffer.copy_(x_local)
        M = self.rows * self.world
        out = torch.empty(M, self.weight.shape[0], dtype=torch.bfloat16, device=self.weight.device)
        self._launch(0, self._x_ptrs, self.K, self.weight, out, None, M, self.weight.shape[0], self.K, self.gathered,
                     self.blk_ready)
        return out

    def forward_nccl(self, x_local: torch.Tensor) -> torch.Tensor:
        full = torch.empty(self.rows * self.world, self.K, dtype=x_local.dtype, device=x_local.device)
        dist.all_gather_into_tensor(full, x_local.contiguous(), group=self.group)
        return full @ self.weight.t()


class RowParallelLinear(_FusedTpBase):
    """``weight``: this rank's [N, K_loc] slice (bf16). Input [M, K_loc] is local; output is this rank's M/world rows."""

    def __init__(self, weight: torch.Tensor, rows_per_rank: int, group=None, **kw):
        super().__init__(group, **kw)
        assert weight.dtype == torch.bfloat16 and weight.is_contiguous() and rows_per_rank % 128 == 0
        self.weight = weight
        self.rows = rows_per_rank
        self.N = weight.shape[0]
        st, hs = _symm(2 * self.world * rows_per_rank * self.N, torch.bfloat16, group)
        self.staging = st
        self._stage_ptrs = self._arr(*[int(p) for p in hs.buffer_ptrs])
        self._keep.append(hs)
        self._sync_setup()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[0] == self.rows * self.world
        out = torch.empty(self.rows, self.N, dtype=torch.bfloat16, device=x.device)
        xp = self._arr(*([x.data_ptr()] * self.world))
        self._launch(1, xp, x.stride(0), self.weight, out, self._stage_ptrs, x.shape[0], self.N, x.shape[1])
        return out

    def forward_nccl(self, x: torch.Tensor) -> torch.Tensor:
        part = x @ self.weight.t()
        out = torch.empty(self.rows, self.N, dtype=part.dtype, device=part.device)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        return out


def shard_weight(w: torch.Tensor, axis: int, rank: int, world: int) -> torch.Tensor:
    """Even split with the remainder going to the first ranks (reference: sharding.rs shard_weight)."""
    n = w.shape[axis]
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    size = base + (1 if rank < rem else 0)
    return w.narrow(axis, start, size).contiguous()
