"""GPU tier: expert parallelism on the device -- the one-launch dispatch planner against the torch planner,
and, where the box has at least two GPUs, the whole expert-parallel layer on two NCCL ranks against the CPU
oracle of the unsharded layer (the reference's own expert-parallel check compares the masked operator with
the full reference, tests/contrib/moe/test_fused_moe.py:35-44,70-81)."""
import os
import socket

import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import ep, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,E,K,world", [(1, 8, 2, 2), (37, 16, 4, 4), (64, 32, 8, 8), (4096, 256, 8, 8), (5000, 64, 6, 32),
                                         (16384, 8, 2, 4)])
def test_plan_kernel_matches_torch_planner(T, E, K, world):
    _, ids = synth.make_routing(T, E, K, "zipf" if E <= 16 else "sigmoid", seed=T)
    ids[0, 0] = -1 if T > 1 else ids[0, 0]                       # an id outside the routing space clamps to rank 0
    pos_w, counts_w, rows_w = ep.plan_positions(ids, E // world, world)
    pos, counts, rows = ep.plan_positions_device(ids.cuda(), E // world, world)
    torch.cuda.synchronize()
    assert torch.equal(pos.cpu(), pos_w)
    assert counts.cpu().tolist() == counts_w.tolist()
    n = int(counts_w.sum())
    assert torch.equal(rows.cpu()[:n].long(), rows_w[:n])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        out = {}
        H, I, K = 512, 256, 4
        E = 16 * world
        El = E // world
        w = synth.make_weights_mxfp4(E, H, I, seed=3)               # every rank can rebuild every expert
        w_loc = tuple(t[rank * El:(rank + 1) * El].to(dev) for t in w)
        for name, T, kw in (("dispatch", 96, dict(exchange="dispatch")),
                            ("gathered", 32, dict(tokens_per_rank=32)),
                            ("dispatch fused combine", 70 + rank, dict(exchange="dispatch", combine="fused"))):
            layer = ep.ExpertParallelMoE(*w_loc, E, rank, world, **kw)
            x = synth.make_hidden(T, H, seed=20 + rank)
            tw, ids = synth.make_routing(T, E, K, "zipf", seed=20 + rank, skew_seed=1)
            y = layer.forward(x.to(dev), tw.to(dev), ids.to(dev))
            torch.cuda.synchronize()
            ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
            out[name] = (orc.cosine(y.cpu(), ref), orc.max_abs(y.cpu(), ref))
        q.put((rank, out))
    except Exception as e:  # noqa: BLE001 - report instead of leaving the parent waiting
        q.put((rank, f"error: {type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_layer_on_two_gpus_matches_the_unsharded_oracle():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    for r in range(world):
        assert isinstance(res[r], dict), res[r]
        for name, (cos, mx) in res[r].items():
            assert cos >= 0.9995 and mx <= 2e-2, (r, name, cos, mx)
