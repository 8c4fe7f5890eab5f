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
     in fp32 in ascending rank (= ascending expert) order by one kernel (`gather_sum`).
The plan of step 2 (`plan_positions`) has no data-dependent shapes, so the counts exchanged in
step 1 are the only values the host reads in a call.

For small batches (decode) the exchange degenerates gracefully into its fixed-shape form: every
rank receives every token (all-gather of rows and routing), runs its local experts on all of them
and the partial outputs are summed back with a reduce-scatter.  No counts, no host read, constant
shapes from step to step -- at T <= `small_batch` tokens per rank the bytes are irrelevant and the
two latencies saved are not.  The fixed-shape form needs the same T on every rank, and every rank
must pick the same form: both are therefore fixed when the layer is built (`tokens_per_rank`,
`exchange`), never read off a rank's own batch.

All collectives are NCCL (`torch.distributed`); device kernels never touch peer memory.  The
integer plumbing (`plan_positions`, and the compact `plan_dispatch` / `scatter_back` pair the tests
compare it with) is backend-agnostic and is exercised with gloo CPU ranks in the tests.
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


def plan_positions(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """Fixed-shape form of `plan_dispatch` (no data-dependent output size, hence no host read):
    returns (pos, counts, rows_padded).  ``pos[t, d]`` is the position of token t inside the
    rank-major send buffer (ascending rank, ascending token within a rank) or -1 when rank d owns none
    of its experts; ``counts[d]`` tokens go to rank d; ``rows_padded[:counts.sum()]`` lists the token
    of every send-buffer position (the tail is padding)."""
    T, K = topk_ids.shape
    dev = topk_ids.device
    dest = torch.div(topk_ids.long(), experts_per_rank, rounding_mode="floor").clamp_(0, world - 1)
    needs = torch.zeros(T, world, dtype=torch.bool, device=dev)
    needs.scatter_(1, dest, True)
    n64 = needs.long()
    counts = n64.sum(dim=0)                                              # [world]
    offs = torch.cumsum(counts, 0) - counts                              # first position of each rank's group
    within = torch.cumsum(n64, 0) - n64                                  # tokens before t bound for the same rank
    pos = torch.where(needs, offs[None, :] + within, torch.full_like(within, -1))
    rows_padded = torch.zeros(T * world + 1, dtype=torch.long, device=dev)
    tok = torch.arange(T, device=dev)[:, None].expand(T, world)
    rows_padded.scatter_(0, torch.where(needs, pos, torch.full_like(pos, T * world)).reshape(-1), tok.reshape(-1))
    return pos.to(torch.int32).contiguous(), counts, rows_padded


def plan_positions_device(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """`plan_positions` as ONE kernel launch behind the C ABI (CUDA tensors): same `pos`, the same `counts`
    (int32 here) and the same defined prefix of `rows` (int32, sized T*world; the tail is unwritten)."""
    import ctypes
    from . import _lib
    T, K = topk_ids.shape
    dev = topk_ids.device
    ids = topk_ids if (topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()) else topk_ids.to(torch.int32).contiguous()
    pos = torch.empty(T, world, dtype=torch.int32, device=dev)
    counts = torch.empty(world, dtype=torch.int32, device=dev)
    rows = torch.empty(max(T * world, 1), dtype=torch.int32, device=dev)
    _lib.check(_lib.lib().b200moe_ep_plan(ctypes.c_void_p(ids.data_ptr()), T, K, experts_per_rank, world,
                                          ctypes.c_void_p(pos.data_ptr()), ctypes.c_void_p(counts.data_ptr()),
                                          ctypes.c_void_p(rows.data_ptr()),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "ep_plan")
    return pos, counts, rows


def gather_sum(rows: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """y[t] = sum_s rows[pos[t, s]] over pos >= 0, fp32 accumulate in slot order, one rounding.
    CUDA tensors go through the library kernel; CPU tensors (the gloo tests of the plumbing) through
    the same arithmetic in torch."""
    T, S = pos.shape
    H = rows.shape[1]
    if rows.is_cuda:
        import ctypes
        from . import _lib
        y = torch.empty(T, H, dtype=rows.dtype, device=rows.device)
        if rows.dtype != torch.bfloat16:
            raise TypeError("gather_sum: bf16 rows expected")
        _lib.check(_lib.lib().b200moe_gather_sum(
            ctypes.c_void_p(rows.data_ptr()), ctypes.c_void_p(pos.data_ptr()), T, S, H, ctypes.c_void_p(y.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "gather_sum")
        return y
    acc = torch.zeros(T, H, dtype=torch.float32)
    for s_ in range(S):
        p = pos[:, s_].long()
        m = p >= 0
        acc[m] += rows[p[m]].float()
    return acc.to(rows.dtype)


class ExpertParallelMoE:
    """One MoE layer sharded by experts.  ``local_fn(x, topk_weight, local_ids) -> y`` computes
    the contribution of this rank's experts for the given rows; by default it is the CUDA
    `fused_moe` on this rank's prepared weights.

    ``exchange``: "dispatch" (all-to-all-v, any per-rank batch sizes), "gathered" (all-gather +
    reduce-scatter, needs ``tokens_per_rank`` tokens on EVERY rank) or "auto": gathered when
    ``tokens_per_rank`` is given and at most ``small_batch``, dispatch otherwise.  The choice is made here,
    from values every rank passes identically, so that no rank can issue a different collective."""

    def __init__(self, w1, w1_scale, w2, w2_scale, num_experts: int, rank: int, world: int,
                 group: Optional[dist.ProcessGroup] = None, local_fn: Optional[Callable] = None,
                 small_batch: int = 512, quant_type=None, dispatch_chunks: Optional[int] = None,
                 exchange: str = "auto", tokens_per_rank: Optional[int] = None, **moe_kwargs):
        if num_experts % world:
            raise ValueError("num_experts must be divisible by the number of ranks")
        if exchange not in ("auto", "gathered", "dispatch"):
            raise ValueError(f"exchange={exchange!r}")
        if exchange == "auto":
            exchange = "gathered" if (tokens_per_rank is not None and tokens_per_rank <= small_batch) else "dispatch"
        if exchange == "gathered" and tokens_per_rank is None:
            raise ValueError("the gathered exchange needs tokens_per_rank: every rank must bring the same token count")
        self.exchange, self.tokens_per_rank = exchange, tokens_per_rank
        self.E, self.rank, self.world, self.group = num_experts, rank, world, group
        self.E_local = num_experts // world
        self.small_batch = small_batch
        self.dispatch_chunks = dispatch_chunks
        if local_fn is None:
            from . import _lib
            from .fused_moe import QuantType, fused_moe, pick_block
            qt = QuantType.per_1x32 if quant_type is None else quant_type
            fmt = _lib.W_FP8_128 if int(qt) == QuantType.per_128x128 else _lib.W_MXFP4
            E_all = num_experts

            def local_fn(x, tw, ids):
                # rows per LOCAL expert = rows * K / E over the whole routing space (most of a row's K ids
                # belong to other ranks), which is what sizes the token tile
                B = pick_block(x.shape[0], ids.shape[1], E_all, fmt)
                return fused_moe(x, w1, w2, tw, ids, quant_type=qt, w1_scale=w1_scale, w2_scale=w2_scale,
                                 block_size_M=B, **moe_kwargs)
        self.local_fn = local_fn
        self.last_local = None      # (rows, weights, local ids) of the latest local call, for measurement
        self.busy_events = None     # set to a list to collect (start, end) CUDA events around the local call
        self.trace = None           # set to a list to collect (phase name, CUDA event) marks of forward_dispatch

    def _mark(self, name, ref):
        if self.trace is not None and ref.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace.append((name, ev))

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
        if self.exchange == "gathered":
            return self.forward_gathered(x, topk_weight, topk_ids)
        return self.forward_dispatch(x, topk_weight, topk_ids)

    def forward_gathered(self, x, topk_weight, topk_ids):
        """Fixed-shape exchange: all-gather rows + routing, local experts over all W*T rows (rows
        routed elsewhere are dropped by the sorter), reduce-scatter of the partial outputs.
        Every rank must call with the same T: the layer's ``tokens_per_rank``, checked here on the host so
        that a stray batch size raises instead of issuing a mismatched collective."""
        T, H = x.shape
        if self.tokens_per_rank is not None and T != self.tokens_per_rank:
            raise ValueError(f"gathered exchange: this rank brought {T} tokens, the layer was built for "
                             f"{self.tokens_per_rank} on every rank (pad the batch, or build the layer with "
                             f"exchange='dispatch')")
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

    def forward_dispatch(self, x: torch.Tensor, topk_weight: torch.Tensor, topk_ids: torch.Tensor,
                         chunks: Optional[int] = None) -> torch.Tensor:
        """All-to-all-v dispatch / local experts / all-to-all-v combine.  One counts exchange and one
        host read per call; everything else is enqueued without synchronisation.

        ``chunks`` > 1 slices the token batch and issues the collectives of all slices asynchronously
        (dispatch of slice c+1 and combine of slice c-1 are in flight while slice c is in the GEMMs).
        Measured on 4 B200 it does not pay (6.36 ms unsliced, 6.72 ms in 2 slices, 7.94 ms in 4 for the
        DeepSeek-V3-shaped layer): the persistent GEMMs occupy every SM, so the collective kernels run
        between them rather than beside them, while every slice streams the local experts' weights
        again and pads its own blocks.  The default is therefore one slice."""
        T, H = x.shape
        K = topk_ids.shape[1]
        W = self.world
        if chunks is None:
            chunks = self.dispatch_chunks or 1
        nch = max(1, min(chunks, T))
        bounds = [T * c // nch for c in range(nch + 1)]
        self._mark("start", x)
        ids32 = topk_ids.to(torch.int32)
        meta = torch.cat([ids32, topk_weight.to(torch.float32).view(torch.int32)], dim=1)    # [T, 2K] int32
        plan = plan_positions_device if x.is_cuda else plan_positions
        plans = [plan(ids32[bounds[c]:bounds[c + 1]], self.E_local, W) for c in range(nch)]
        send_counts = (plans[0][1].reshape(W, 1) if nch == 1 else
                       torch.stack([p[1] for p in plans], dim=1)).contiguous()              # [W, nch]
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # the only host read of the call: all_to_all_single takes Python split sizes
        self._mark("planned", x)
        counts = torch.stack([send_counts, recv_counts]).cpu().tolist()
        self._mark("counts_on_host", x)

        inflight = []
        for c in range(nch):
            s_splits = [counts[0][d][c] for d in range(W)]
            r_splits = [counts[1][d][c] for d in range(W)]
            rows = plans[c][2][:sum(s_splits)]
            if bounds[c]:
                rows = rows + bounds[c]
            n_recv = sum(r_splits)
            x_recv = torch.empty(n_recv, H, dtype=x.dtype, device=x.device)
            m_recv = torch.empty(n_recv, 2 * K, dtype=torch.int32, device=x.device)
            wx = dist.all_to_all_single(x_recv, x[rows], r_splits, s_splits, group=self.group, async_op=True)
            wm = dist.all_to_all_single(m_recv, meta[rows], r_splits, s_splits, group=self.group, async_op=True)
            inflight.append((len(rows), s_splits, r_splits, x_recv, m_recv, wx, wm))
        self._mark("dispatch_issued", x)

        back = []
        for n_send, s_splits, r_splits, x_recv, m_recv, wx, wm in inflight:
            wx.wait()
            wm.wait()
            self._mark("dispatch_done", x)
            local_ids = (m_recv[:, :K] - self.rank * self.E_local).contiguous()   # foreign experts land outside [0, E_local)
            tw_recv = m_recv[:, K:].contiguous().view(torch.float32)
            y_part = self._local(x_recv, tw_recv, local_ids) if x_recv.shape[0] else x_recv
            self._mark("local_done", x)
            y_back = torch.empty(n_send, H, dtype=x.dtype, device=x.device)
            wy = dist.all_to_all_single(y_back, y_part.contiguous(), s_splits, r_splits, group=self.group, async_op=True)
            back.append((y_back, wy))
        y = torch.empty(T, H, dtype=x.dtype, device=x.device)
        for c, (y_back, wy) in enumerate(back):
            wy.wait()
            self._mark("combine_done", x)
            y[bounds[c]:bounds[c + 1]] = gather_sum(y_back, plans[c][0])
        self._mark("end", x)
        return y
