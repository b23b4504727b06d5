"""Column-parallel sharding of one GEMM over the GPUs of a node (no reduction).

`Y = act(X @ W)` with W split along N: rank r keeps all of X and the contiguous column block
`W[:, r*N/g:(r+1)*N/g]` re-packed as a dense `[K, N/g]` matrix, and computes its own `[M, N/g]`
block of Y. Bias and activation are column-local, so the epilogue needs no communication. K is
never split: that would need a reduce-scatter and would break the saturate-once rule of the I8
path and bitwise determinism.

The optional all-gather follows numr's `Communicator::all_gather(send, recv, count, dtype)`
(src/runtime/communicator/traits.rs:82-94, NCCL call at src/runtime/cuda/communicator.rs:146-166):
the collective concatenates the ranks' buffers along the leading dimension, so the gathered
`[g, M, N/g]` staging buffer is re-interleaved into row-major `[M, N]` afterwards.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def column_range(n_total: int, world: int, rank: int) -> slice:
    """Columns of W (and of Y) that `rank` owns; N must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    if n_total % world != 0:
        raise ValueError(f"N = {n_total} does not split evenly over {world} ranks")
    per = n_total // world
    return slice(rank * per, (rank + 1) * per)


def pack_weight_shard(w: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Dense `[K, N/g]` copy of this rank's column block of W `[K, N]` (the layout the launchers read)."""
    if w.dim() != 2:
        raise ValueError("W must be [K, N]")
    return w[:, column_range(w.shape[1], world, rank)].contiguous()


def unshard_columns(blocks) -> torch.Tensor:
    """Row-major `[M, N]` from the ranks' `[M, N/g]` blocks, in rank order."""
    return torch.cat(list(blocks), dim=1)


def all_gather_columns(y_shard: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers the `[M, N/g]` blocks and returns the full row-major `[M, N]` on every rank.

    Works on any backend (NCCL for CUDA tensors, gloo for CPU tensors)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_shard
    y_shard = y_shard.contiguous()
    m, per = y_shard.shape
    staging = torch.empty((world * m, per), dtype=y_shard.dtype, device=y_shard.device)
    dist.all_gather_into_tensor(staging, y_shard, group=group)
    # [g*M, N/g] = [g, M, N/g] -> [M, g, N/g] -> [M, N]
    return staging.view(world, m, per).permute(1, 0, 2).reshape(m, world * per)


class GatheredOutput:
    """The row-major `[M, N]` result of a column-sharded GEMM, one copy per rank, each rank's copy
    mapped into every other rank's address space so that the GEMM's epilogue can store its tiles
    into all of them (`CudaClient.matmul_activation_allgather`): the all-gather happens inside the
    kernel, tile by tile, and lands row-major (no `[g, M, N/g]` staging, no re-interleave).

    The mappings come from torch's symmetric memory (device memory and rendezvous only). `barrier()`
    orders the ranks on the current stream: call it after the fused GEMM before anyone reads the
    buffer, and again before the next fused GEMM overwrites it. Multicast objects are not used."""

    def __init__(self, m: int, n_total: int, dtype, device, group=None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._handle = None
        if self.world == 1:
            self.tensor = torch.empty((m, n_total), dtype=dtype, device=device)
            self.ptrs = [self.tensor.data_ptr()]
        else:
            import os
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            self.tensor = symm.empty((m, n_total), dtype=dtype, device=device)
            self._handle = symm.rendezvous(self.tensor, group if group is not None else dist.group.WORLD)
            self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
            assert self.ptrs[self.rank] == self.tensor.data_ptr()

    @classmethod
    def emulated(cls, buffers, rank: int):
        """Several "ranks" on one GPU: `buffers` are the ranks' `[M, N]` tensors, all local. For tests
        of the kernel's store pattern where only one GPU is at hand."""
        self = cls.__new__(cls)
        self.world, self.rank, self._handle = len(buffers), rank, None
        self.tensor = buffers[rank]
        self.ptrs = [b.data_ptr() for b in buffers]
        return self

    def barrier(self):
        """All ranks have passed this point of their current stream (device-side, over NVLink signals)."""
        if self._handle is not None:
            self._handle.barrier()


def sharded_matmul_activation(client, x: torch.Tensor, w_shard: torch.Tensor, activation, bias_shard=None):
    """This rank's block: `act(X @ W_r (+ bias_r))` through the client's fused ops."""
    from .client import GemmActivation
    if bias_shard is not None:
        return client.matmul_bias_activation(x, w_shard, bias_shard, activation)
    if activation == GemmActivation.NONE:
        return client.matmul(x, w_shard)
    return client.matmul_activation(x, w_shard, activation)
