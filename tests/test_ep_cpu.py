"""CPU tier: the expert-parallel dispatch/combine plumbing with gloo ranks (world size 2 and 4),
including a rank that never joins the exchange (failure detection by timeout, no GPU involved)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as orc
from pyhip_b200 import ep, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fail_rank, q, small_batch=0, chunks=1, uneven=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8 if fail_rank is not None else 60))
    try:
        T, H, I, E, K = 24, 128, 64, 8, 3
        T_agreed = T
        if uneven:
            T += rank               # this rank's batch differs from what the layer was built for
        w = synth.make_weights_mxfp4(E, H, I, seed=2)
        w1, w2 = orc.dequant_mxfp4(w[0], w[1]), orc.dequant_mxfp4(w[2], w[3])
        x = synth.make_hidden(T, H, seed=10 + rank)
        tw, ids = synth.make_routing(T, E, K, "zipf", seed=10 + rank)
        El = E // world
        lo = rank * El

        def local_fn(xr, twr, ids_local):
            return orc.torch_moe_oracle(xr, w1[lo:lo + El], w2[lo:lo + El], twr, ids_local)

        layer = ep.ExpertParallelMoE(None, None, None, None, E, rank, world, local_fn=local_fn,
                                     small_batch=small_batch, dispatch_chunks=chunks, tokens_per_rank=T_agreed)
        if fail_rank == rank:
            q.put((rank, "skipped"))
            return
        try:
            y = layer.forward(x, tw, ids)
        except Exception as e:  # noqa: BLE001 - the surviving rank must see an error, not hang
            q.put((rank, "error:" + type(e).__name__))
            return
        ref = orc.torch_moe_oracle(x, w1, w2, tw, ids)
        q.put((rank, (orc.cosine(y, ref), orc.max_abs(y, ref))))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _spawn(world, fail_rank=None, small_batch=0, chunks=1, uneven=False):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, q, small_batch, chunks, uneven))
             for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


def test_plan_dispatch_groups_tokens_once_per_rank():
    ids = torch.tensor([[0, 1, 7], [4, 5, 6], [3, 4, 0]], dtype=torch.int32)
    rows, counts = ep.plan_dispatch(ids, 4, 2)
    assert counts.tolist() == [2, 3]
    assert rows.tolist() == [0, 2, 0, 1, 2]
    y = ep.scatter_back(torch.ones(5, 4), rows, 3)
    assert y[:, 0].tolist() == [2.0, 1.0, 2.0]


@pytest.mark.parametrize("T,E,K,world", [(37, 16, 4, 4), (5, 8, 2, 2), (64, 32, 8, 8)])
def test_plan_positions_matches_plan_dispatch(T, E, K, world):
    """The fixed-shape planner (no host read) lists the same rows in the same order as the compact one,
    and its position table inverts that list."""
    _, ids = synth.make_routing(T, E, K, "zipf", seed=T)
    rows, counts = ep.plan_dispatch(ids, E // world, world)
    pos, counts2, rows_padded = ep.plan_positions(ids, E // world, world)
    assert counts.tolist() == counts2.tolist()
    n = int(counts.sum())
    assert rows_padded[:n].tolist() == rows.tolist()
    for t in range(T):
        for d in range(world):
            p_ = int(pos[t, d])
            owns = bool(((ids[t] // (E // world)) == d).any())
            assert (p_ >= 0) == owns
            if owns:
                assert int(rows[p_]) == t
    y_rows = torch.randn(n, 16).to(torch.bfloat16)
    assert torch.equal(ep.gather_sum(y_rows, pos), ep.scatter_back(y_rows, rows, T))


@pytest.mark.parametrize("world,small_batch,chunks", [(2, 0, 1), (4, 0, 1), (2, 512, 1), (2, 0, 3), (4, 0, 2)])
def test_expert_parallel_matches_single_process_oracle(world, small_batch, chunks):
    """small_batch=0 forces the all-to-all-v dispatch/combine (in `chunks` pipelined slices), 512 the
    gathered fixed-shape form."""
    res = _spawn(world, small_batch=small_batch, chunks=chunks)
    for r in range(world):
        cos, mx = res[r]
        assert cos > 0.9999 and mx < 5e-3, (r, cos, mx)


def test_one_expert_per_rank_on_eight_ranks():
    """The Mixtral-shaped configuration at 8 GPUs leaves ONE expert per rank: every local id is 0 and most of a
    token's ids belong to other ranks."""
    res = _spawn(8)
    for r in range(8):
        cos, mx = res[r]
        assert cos > 0.9999 and mx < 5e-3, (r, cos, mx)


def test_rank_that_never_joins_is_detected_by_timeout():
    res = _spawn(2, fail_rank=1)
    assert res[1] == "skipped"
    assert isinstance(res[0], str) and res[0].startswith("error:")


def test_unequal_batches_raise_on_the_host_in_the_gathered_form_and_work_in_the_dispatch_form():
    """The exchange form is fixed when the layer is built, from values all ranks share.  A rank whose batch
    differs from the agreed `tokens_per_rank` gets a ValueError before any collective is issued in the
    fixed-shape (gathered) form -- rank 0, whose batch matches, sees its peer missing as a timeout/error
    instead of summing the wrong rows -- while the all-to-all-v form takes unequal batches as they come."""
    res = _spawn(2, small_batch=512, uneven=True, fail_rank=-1)       # gathered; fail_rank=-1 only shortens the timeout
    assert res[1] == "error:ValueError"
    assert isinstance(res[0], str) and res[0].startswith("error:")
    res = _spawn(2, small_batch=0, uneven=True)                       # dispatch
    for r in range(2):
        cos, mx = res[r]
        assert cos > 0.9999 and mx < 5e-3, (r, cos, mx)


def test_exchange_choice_needs_agreed_values():
    with pytest.raises(ValueError):
        ep.ExpertParallelMoE(None, None, None, None, 8, 0, 2, local_fn=lambda *a: None, exchange="gathered")
    layer = ep.ExpertParallelMoE(None, None, None, None, 8, 0, 2, local_fn=lambda *a: None)
    assert layer.exchange == "dispatch"                               # no agreed token count: the form that needs none
    layer = ep.ExpertParallelMoE(None, None, None, None, 8, 0, 2, local_fn=lambda *a: None, tokens_per_rank=64)
    assert layer.exchange == "gathered"
    layer = ep.ExpertParallelMoE(None, None, None, None, 8, 0, 2, local_fn=lambda *a: None, tokens_per_rank=4096)
    assert layer.exchange == "dispatch"
