"""Multi-GPU plumbing for the two ways the path shards (one process per GPU, ``torch.distributed``):

* tensor parallel: the rows of a weight matrix are independent (each row is its own run of blocks), so
  rank r keeps rows ``row_shard(n_out, world, r)``, every rank multiplies the same activations by its
  shard, and one all-gather along the output columns rebuilds ``y`` (``gather_columns``);
* expert parallel: rank r keeps the experts ``expert_shard(n_experts, world, r)``; tokens start sharded
  over the ranks, and each (token, route) pair travels to the rank that owns the expert and back
  (``ExpertParallel``: counts first, then the payload, both with all-to-all).

The reference has a single device and no collective at all, so parity is defined against the
single-device result: sharded dense outputs are bit-identical per column (the same kernel computes the
same row), and expert-parallel outputs are bit-identical too because the combine keeps the route order.
Everything here works on CPU tensors with the ``gloo`` backend (the host-logic tests) and on CUDA
tensors with ``nccl``; the local compute is passed in as a callable.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def row_shard(n_out: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Rows ``[r0, r1)`` of rank ``rank``: equal contiguous shares in units of ``multiple`` rows (FP8
    block scales need 128), the remainder going to the last ranks that still have rows."""
    units = -(-n_out // multiple)
    per = -(-units // world)
    r0 = min(n_out, rank * per * multiple)
    r1 = min(n_out, (rank + 1) * per * multiple)
    return r0, r1


def expert_shard(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    per = -(-n_experts // world)
    return min(n_experts, rank * per), min(n_experts, (rank + 1) * per)


def gather_columns(y_local: torch.Tensor, n_out: int, group=None) -> torch.Tensor:
    """All-gather of row-sharded outputs: ``y_local`` is ``[t, n_local]`` (equal ``n_local`` on every rank,
    zero-padded on the last one if needed); returns ``[t, n_out]``."""
    world = dist.get_world_size(group)
    t, n_local = y_local.shape
    buf = torch.empty((world * t, n_local), dtype=y_local.dtype, device=y_local.device)  # rank-major concatenation
    dist.all_gather_into_tensor(buf, y_local.contiguous(), group=group)
    return buf.reshape(world, t, n_local).permute(1, 0, 2).reshape(t, world * n_local)[:, :n_out]


class ExpertParallel:
    """Dispatch / combine of an expert-parallel MoE layer.

    ``local_experts(x_rows, expert_ids) -> o_rows`` computes, for every received row i, the full expert
    ``down(act(gate x) * up x)`` of LOCAL expert ``expert_ids[i]`` (an index into this rank's shard).
    """

    def __init__(self, n_experts: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_experts = n_experts
        self.per = -(-n_experts // self.world)

    def forward(self, x: torch.Tensor, route_ids: torch.Tensor, route_w: torch.Tensor, y: torch.Tensor,
                local_experts: Callable[[torch.Tensor, torch.Tensor], torch.Tensor]) -> torch.Tensor:
        """``y[i] += sum_j w_ij * expert_{ids_ij}(x_i)`` for this rank's tokens ``x`` ``[t, h]``; routes are ``[t, k]``."""
        t, k = route_ids.shape
        h = x.shape[1]
        dev = x.device
        flat_e = route_ids.reshape(-1).to(torch.int64)
        owner = flat_e // self.per
        order = torch.argsort(owner, stable=True)          # pairs grouped by destination rank, token order kept
        send_counts = torch.bincount(owner, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)   # counts first
        s_split, r_split = send_counts.tolist(), recv_counts.tolist()
        tok = torch.arange(t, device=dev).repeat_interleave(k)[order]
        send_x = x[tok].contiguous()
        send_e = (flat_e[order] - owner[order] * self.per).to(torch.int32).contiguous()
        n_recv = int(sum(r_split))
        recv_x = torch.empty((n_recv, h), dtype=x.dtype, device=dev)
        recv_e = torch.empty((n_recv,), dtype=torch.int32, device=dev)
        dist.all_to_all_single(recv_x, send_x, r_split, s_split, group=self.group)   # payload second
        dist.all_to_all_single(recv_e, send_e, r_split, s_split, group=self.group)
        o = local_experts(recv_x, recv_e) if n_recv else torch.empty((0, h), dtype=y.dtype, device=dev)
        back = torch.empty((t * k, h), dtype=o.dtype, device=dev)
        dist.all_to_all_single(back, o.contiguous(), s_split, r_split, group=self.group)   # combine: the way back
        per_pair = torch.empty_like(back)
        per_pair[order] = back                                # back to (token, route) order
        per_pair = per_pair.reshape(t, k, h)
        for j in range(k):                                    # axpy in route order (src/cuda.rs:319-330)
            y += route_w[:, j : j + 1].to(y.dtype) * per_pair[:, j, :].to(y.dtype)
        return y
