"""Expert-parallel execution of the MoE layer across the GPUs of one box.

The reference has no dispatch/combine: expert parallelism exists there only as an input
convention (`expert_mask`, src/contrib/fused_moe.py:134,210-212) and a single-process simulation
(tests/contrib/moe/test_fused_moe.py:35-44,70-81).  Here rank g owns the contiguous expert range
[g*E/G, (g+1)*E/G) -- the same convention as that mask -- and the exchange is:

  1. counts all-to-all ([G] integers),
  2. dispatch all-to-all-v: each token row travels ONCE to every rank that owns at least one of
     its experts, together with its K routing ids and weights,
  3. the local fused-MoE on the received rows (ids re-based to the local range; ids owned by
     other ranks fall outside [0, E_local) and are dropped by the sorter),
  4. combine all-to-all-v of the per-rank partial outputs back to the source rank, summed there
     in fp32 in ascending rank (= ascending expert) order.

For small batches (decode) the exchange degenerates gracefully into its fixed-shape form: every
rank receives every token (all-gather of rows and routing), runs its local experts on all of them
and the partial outputs are summed back with a reduce-scatter.  No counts, no host read, constant
shapes from step to step -- at T <= `small_batch` tokens per rank the bytes are irrelevant and the
two latencies saved are not.

All collectives are NCCL (`torch.distributed`); device kernels never touch peer memory.  The
integer plumbing (`plan_dispatch`, `scatter_back`) is backend-agnostic and is exercised with gloo
CPU ranks in the tests.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """Which token goes to which rank.

    Returns (send_rows, send_counts): ``send_rows`` lists token indices grouped by destination
    rank (ascending rank, ascending token inside a rank); ``send_counts[d]`` is the number of
    tokens bound for rank d."""
    T, K = topk_ids.shape
    dest = torch.div(topk_ids.long(), experts_per_rank, rounding_mode="floor").clamp_(0, world - 1)   # [T, K]
    needs = torch.zeros(T, world, dtype=torch.bool, device=topk_ids.device)
    needs.scatter_(1, dest, True)
    needs_t = needs.t().contiguous()                       # [world, T]
    send_counts = needs_t.sum(dim=1)
    send_rows = needs_t.nonzero(as_tuple=False)[:, 1]       # row-major: grouped by rank, token ascending
    return send_rows, send_counts


def scatter_back(y_back: torch.Tensor, send_rows: torch.Tensor, T: int) -> torch.Tensor:
    """Sum the partial outputs returned by the owner ranks into token order (fp32 accumulate,
    deterministic: index_add_ walks the rank-grouped rows in order)."""
    acc = torch.zeros(T, y_back.shape[1], dtype=torch.float32, device=y_back.device)
    acc.index_add_(0, send_rows, y_back.float())
    return acc.to(y_back.dtype)


class ExpertParallelMoE:
    """One MoE layer sharded by experts.  ``local_fn(x, topk_weight, local_ids) -> y`` computes
    the contribution of this rank's experts for the given rows; by default it is the CUDA
    `fused_moe` on this rank's prepared weights."""

    def __init__(self, w1, w1_scale, w2, w2_scale, num_experts: int, rank: int, world: int,
                 group: Optional[dist.ProcessGroup] = None, local_fn: Optional[Callable] = None,
                 small_batch: int = 512, quant_type=None):
        if num_experts % world:
            raise ValueError("num_experts must be divisible by the number of ranks")
        self.E, self.rank, self.world, self.group = num_experts, rank, world, group
        self.E_local = num_experts // world
        self.small_batch = small_batch
        if local_fn is None:
            from .fused_moe import QuantType, fused_moe
            qt = QuantType.per_1x32 if quant_type is None else quant_type

            def local_fn(x, tw, ids):
                return fused_moe(x, w1, w2, tw, ids, quant_type=qt, w1_scale=w1_scale, w2_scale=w2_scale)
        self.local_fn = local_fn
        self.last_local = None      # (rows, weights, local ids) of the latest local call, for measurement
        self.busy_events = None     # set to a list to collect (start, end) CUDA events around the local call

    def _local(self, x, tw, ids):
        self.last_local = (x, tw, ids)
        if self.busy_events is None:
            return self.local_fn(x, tw, ids)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        y = self.local_fn(x, tw, ids)
        e1.record()
        self.busy_events.append((e0, e1))
        return y

    def _a2a(self, out, inp, out_splits, in_splits):
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    def forward(self, x: torch.Tensor, topk_weight: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        if x.shape[0] <= self.small_batch:
            return self.forward_gathered(x, topk_weight, topk_ids)
        return self.forward_dispatch(x, topk_weight, topk_ids)

    def forward_gathered(self, x, topk_weight, topk_ids):
        """Fixed-shape exchange: all-gather rows + routing, local experts over all W*T rows (rows
        routed elsewhere are dropped by the sorter), reduce-scatter of the partial outputs.
        Every rank must call with the same T."""
        T, H = x.shape
        K = topk_ids.shape[1]
        W = self.world
        x_all = torch.empty(W * T, H, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
        meta = torch.cat([topk_ids.to(torch.int32), topk_weight.to(torch.float32).view(torch.int32)], dim=1)
        meta_all = torch.empty(W * T, 2 * K, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(meta_all, meta.contiguous(), group=self.group)
        local_ids = (meta_all[:, :K] - self.rank * self.E_local).contiguous()
        tw_all = meta_all[:, K:].contiguous().view(torch.float32)
        y_part = self._local(x_all, tw_all, local_ids)
        y = torch.empty(T, H, dtype=x.dtype, device=x.device)
        if dist.get_backend(self.group) == "nccl":
            dist.reduce_scatter_tensor(y, y_part.contiguous(), op=dist.ReduceOp.SUM, group=self.group)
        else:                                   # gloo has no reduce-scatter: sum everywhere, keep own slice
            acc = y_part.float()
            dist.all_reduce(acc, group=self.group)
            y.copy_(acc[self.rank * T:(self.rank + 1) * T])
        return y

    def forward_dispatch(self, x: torch.Tensor, topk_weight: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        K = topk_ids.shape[1]
        send_rows, send_counts = plan_dispatch(topk_ids, self.E_local, self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # one host read of both count vectors: all_to_all_single takes Python split sizes
        counts = torch.stack([send_counts, recv_counts]).cpu().tolist()
        s_splits, r_splits = counts[0], counts[1]
        n_recv = sum(r_splits)

        x_recv = torch.empty(n_recv, H, dtype=x.dtype, device=x.device)
        ids_recv = torch.empty(n_recv, K, dtype=topk_ids.dtype, device=x.device)
        tw_recv = torch.empty(n_recv, K, dtype=topk_weight.dtype, device=x.device)
        self._a2a(x_recv, x[send_rows].contiguous(), r_splits, s_splits)
        self._a2a(ids_recv, topk_ids[send_rows].contiguous(), r_splits, s_splits)
        self._a2a(tw_recv, topk_weight[send_rows].contiguous(), r_splits, s_splits)

        local_ids = ids_recv - self.rank * self.E_local      # foreign experts land outside [0, E_local)
        y_part = self._local(x_recv, tw_recv, local_ids) if n_recv else x_recv
        y_back = torch.empty(len(send_rows), H, dtype=x.dtype, device=x.device)
        self._a2a(y_back, y_part.contiguous(), s_splits, r_splits)
        return scatter_back(y_back, send_rows, T)
