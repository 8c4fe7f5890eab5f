"""GPU tier: the sort/align kernel is bit-exact with the oracle over the defined prefix."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import moe_sorting, synth

pytestmark = pytest.mark.gpu


def _run(ids, tw, E, B, mask=None):
    dev = torch.device("cuda:0")
    m = None if mask is None else torch.tensor(mask, dtype=torch.int32, device=dev)
    s_ids, s_w, s_e, nv, out = moe_sorting(ids.to(dev), tw.to(dev), E, 8, torch.bfloat16, B, expert_mask=m)
    torch.cuda.synchronize()
    return (s_ids.cpu().numpy().view(np.uint32), s_w.cpu().numpy(), s_e.cpu().numpy(), nv.cpu().numpy(), out)


def _check(ids, tw, E, B, mask=None):
    got = _run(ids, tw, E, B, mask)
    exp = orc.moe_sorting_oracle(ids, tw, E, B, expert_mask=mask)
    n = int(exp[3][0])
    assert got[3].tolist() == exp[3].tolist()
    assert np.array_equal(got[0][:n], exp[0][:n])
    assert np.array_equal(got[1][:n].view(np.uint32), exp[1][:n].view(np.uint32))
    assert np.array_equal(got[2][:n // B], exp[2][:n // B])
    assert got[4].abs().sum().item() == 0


@pytest.mark.parametrize("B", [16, 32, 64, 128, 256])
def test_tiny_config_all_block_sizes(B):
    c = synth.CONFIGS["tiny"]
    tw, ids = synth.make_routing(c.T, c.E, c.K)
    _check(ids, tw, c.E, B)


@pytest.mark.parametrize("T,E,K,routing", [(1, 128, 4, "softmax"), (8, 128, 4, "softmax"), (64, 128, 4, "softmax"),
                                           (300, 16, 4, "zipf"), (2048, 8, 2, "zipf"), (1000, 256, 8, "sigmoid"),
                                           (8192, 128, 4, "softmax"), (16384, 8, 2, "zipf")])
def test_shapes_and_skew(T, E, K, routing):
    tw, ids = synth.make_routing(T, E, K, routing, seed=T)
    _check(ids, tw, E, 32 if T <= 64 else 128)


def test_expert_mask_local_ids():
    ids = torch.tensor([[0, 3, 5], [2, 3, 5], [1, 3, 5], [1, 2, 3], [1, 3, 5]], dtype=torch.int32)
    tw = torch.arange(15, dtype=torch.float32).reshape(5, 3) + 1
    _check(ids, tw, 6, 4)
    _check(ids, tw, 6, 4, mask=[1, 0, 1, 1, 0, 1])
    got = _run(ids, tw, 6, 4, mask=[1, 0, 1, 1, 0, 1])
    assert got[3][0] == 20 and got[2][:5].tolist() == [0, 1, 2, 2, 3]


def test_all_tokens_to_one_expert_and_empty_experts():
    T, E, K = 257, 64, 1
    ids = torch.full((T, K), 63, dtype=torch.int32)
    tw = torch.rand(T, K)
    _check(ids, tw, E, 32)


@pytest.mark.parametrize("T,n", [(64, 40), (64, 0), (300, 299), (8, 1)])
def test_num_local_tokens_sorts_only_the_live_prefix(T, n):
    """With a device-side live count the sorter treats the batch as its first n tokens
    (src/contrib/fused_moe.py:48-49,63): same rows, same order; only the sentinel keeps the padded T."""
    E, K, B = 16, 4, 32
    tw, ids = synth.make_routing(T, E, K, seed=T + n)
    dev = torch.device("cuda:0")
    nl = torch.tensor([n], dtype=torch.int32, device=dev)
    s_ids, s_w, s_e, nv, _ = moe_sorting(ids.to(dev), tw.to(dev), E, 8, torch.bfloat16, B, num_local_tokens=nl)
    torch.cuda.synchronize()
    exp = orc.moe_sorting_oracle(ids[:n], tw[:n], E, B)
    L = int(exp[3][0])
    assert nv.cpu().tolist() == [L, n]
    got_ids = s_ids.cpu().numpy().view(np.uint32)[:L]
    live = (exp[0][:L] >> 24) < K
    assert np.array_equal(got_ids[live], exp[0][:L][live])
    assert np.all(got_ids[~live] == ((K << 24) | T))
    assert np.array_equal(s_w.cpu().numpy()[:L].view(np.uint32), exp[1][:L].view(np.uint32))
    assert np.array_equal(s_e.cpu().numpy()[:L // B], exp[2][:L // B])


def test_reference_golden_sort_vectors_on_the_device():
    """The fixture holds the outputs of the reference's own moe_sorting_ref (lifted out of
    src/contrib/fused_moe.py:56-100 and run on CPU, tests/golden/make_golden.py) for a block size of 256:
    the device sort must reproduce its defined prefix bit for bit."""
    import pathlib
    g = np.load(pathlib.Path(__file__).parent / "golden" / "sorting_b256.npz")
    ids, tw = torch.from_numpy(g["topk_ids"]), torch.from_numpy(g["topk_weight"])
    E, B, n = int(g["E"]), int(g["B"]), int(g["num_valid"])
    got = _run(ids, tw, E, B)
    assert got[3].tolist() == [n, ids.shape[0]]
    assert np.array_equal(got[0][:n], g["sorted_ids"])
    assert np.array_equal(got[1][:n].view(np.uint32), g["sorted_weights"].view(np.uint32))
    assert np.array_equal(got[2][:n // B], g["sorted_expert_ids"])
