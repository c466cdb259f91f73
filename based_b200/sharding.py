"""Sharding across ranks (one process per GPU): batch x heads shards, and head-sharded tensor parallelism.

Every (batch, head) pair is independent in all kernels of this path, so N GPUs need no
data-path collective: each rank takes a contiguous slice of the batch (the unit the full
model shards by; heads of one sample stay together so a sample's mixer output is complete
on one rank).  The only cross-rank step is the timing reduction of the benchmark.
"""
from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [start, end) of `total` units for `rank`; the first `total % world` ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(values, device) -> list:
    """Element-wise max of a list of floats over all ranks (identity when not distributed)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def sum_over_ranks(values, device) -> list:
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.tolist()


# --------------------------------------------------------------------------- head-sharded tensor parallelism
# The reference mixers have no tensor-parallel support (LinearAttention takes no process group,
# based/models/mixers/linear_attention.py:78-90).  This variant follows the reference's own
# RowParallelLinear (based/ops/fused_dense.py:205-246): q/k/v projections column-parallel (each rank owns
# num_heads / world heads and their slice of the recurrent state), out_proj row-parallel, and ONE all-reduce of
# the [B, L, d_model] output (NCCL over NVLink on GPUs).  Nothing inside the kernels crosses ranks.

def head_slice(num_heads: int, rank: int, world: int) -> Tuple[int, int]:
    if num_heads % world != 0:
        raise ValueError(f"num_heads={num_heads} is not divisible by the tensor-parallel size {world}")
    per = num_heads // world
    return rank * per, (rank + 1) * per


def shard_linear_attention_state_dict(full: dict, num_heads: int, feature_dim: int, head_dim: int,
                                      rank: int, world: int, prefix: str = "") -> dict:
    """Slice a full LinearAttention state_dict (reference parameter names) for one tensor-parallel rank."""
    h0, h1 = head_slice(num_heads, rank, world)
    out = {}
    out[prefix + "proj_q.weight"] = full[prefix + "proj_q.weight"][h0 * feature_dim:h1 * feature_dim].clone()
    out[prefix + "proj_k.weight"] = full[prefix + "proj_k.weight"][h0 * feature_dim:h1 * feature_dim].clone()
    out[prefix + "proj_v.weight"] = full[prefix + "proj_v.weight"][h0 * head_dim:h1 * head_dim].clone()
    out[prefix + "out_proj.weight"] = full[prefix + "out_proj.weight"][:, h0 * head_dim:h1 * head_dim].clone()
    return out


def shard_sliding_attention_state_dict(full: dict, num_heads: int, head_dim: int, rank: int, world: int,
                                       prefix: str = "") -> dict:
    """Slice a full SlidingAttention state_dict (Wqkv rows are ordered (three, head, dim),
    based/models/mixers/slide_attention.py:546) for one tensor-parallel rank."""
    h0, h1 = head_slice(num_heads, rank, world)
    w = full[prefix + "Wqkv.weight"]
    d_model = w.shape[1]
    w3 = w.view(3, num_heads, head_dim, d_model)[:, h0:h1].reshape(3 * (h1 - h0) * head_dim, d_model)
    out = {prefix + "Wqkv.weight": w3.clone(),
           prefix + "out_proj.weight": full[prefix + "out_proj.weight"][:, h0 * head_dim:h1 * head_dim].clone()}
    if prefix + "Wqkv.bias" in full:
        b = full[prefix + "Wqkv.bias"].view(3, num_heads, head_dim)[:, h0:h1].reshape(-1)
        out[prefix + "Wqkv.bias"] = b.clone()
    if prefix + "out_proj.bias" in full and h0 == 0:
        out[prefix + "out_proj.bias"] = full[prefix + "out_proj.bias"].clone()  # row-parallel: added once, by the rank owning head 0
    return out


def all_reduce_sum_(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the tensor-parallel group (identity for a group of one / no group)."""
    if group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


# --------------------------------------------------------------------------- fused out_proj + all-reduce (decode steps)
class PeerWorkspace:
    """One device buffer per rank of a process group, each mapped into every rank's address space, so that a kernel
    can store into its peers' buffers over NVLink.  The mapping is torch's: symmetric memory
    (``torch.distributed._symmetric_memory``) — allocation, handle exchange through the group's store and mapping are
    its job; this class only keeps the tensor alive and hands out the addresses.  Creating one is a collective."""

    def __init__(self, nbytes: int, group, device):
        import os

        import torch.distributed._symmetric_memory as symm
        # the kernels here use plain peer loads / stores only: no NVLink multicast object needs to be bound
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.tensor = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.tensor.data_ptr():
            raise RuntimeError("symmetric memory returned an unexpected address table")


class FusedRowParallel:
    """Decode-step ``all_reduce(x W^T)`` of a row-parallel projection as ONE kernel per rank
    (:func:`based_b200.ops.tp_outproj_allreduce`).  Built lazily by the mixers on their first decode step; the set-up is
    a collective (every rank of the group must reach it), and so is every call."""

    def __init__(self, n_out: int, max_rows: int, group, device):
        from . import ops
        self.max_rows, self.n_out = int(max_rows), int(n_out)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.ws = PeerWorkspace(ops.tp_outproj_workspace_bytes(self.world, self.max_rows, self.n_out), group, device)
        ops.tp_outproj_workspace_init_(self.ws.tensor)
        torch.cuda.synchronize(device)
        dist.barrier(group)            # nobody pushes into a workspace that its owner is still clearing

    def __call__(self, x, weight, bias=None):
        from . import ops
        return ops.tp_outproj_allreduce(x, weight, bias, self.ws.ptrs, self.max_rows, self.rank, self.world)


def row_parallel_decode_linear(owner, x, weight, bias, group, max_rows: int = 64):
    """``all_reduce(x W^T (+ bias))`` for a decode step of a row-parallel projection.  With ``owner.fused_allreduce`` set,
    bf16 tensors, no bias and at most ``max_rows`` rows it is the one-kernel form (the :class:`FusedRowParallel` is built
    on first use and kept on ``owner``); otherwise a GEMM followed by an NCCL all-reduce."""
    from . import ops
    rows = x.numel() // x.shape[-1] if x.numel() else 0
    fused_ok = (group is not None and getattr(owner, "fused_allreduce", False) and bias is None and x.is_cuda
                and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= max_rows
                and x.shape[-1] % 32 == 0 and weight.shape[0] % 8 == 0 and weight.is_contiguous()
                and not torch.is_grad_enabled() and dist.get_world_size(group) <= 8)
    if not fused_ok:
        return all_reduce_sum_(ops.linear(x, weight, bias), group)
    fused = getattr(owner, "_fused_row_parallel", None)
    if fused is None:
        fused = FusedRowParallel(weight.shape[0], max_rows, group, x.device)
        owner._fused_row_parallel = fused
    return fused(x, weight)
