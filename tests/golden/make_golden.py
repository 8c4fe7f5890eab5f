"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own functions.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's test module cannot be imported (it imports ROCm-only packages at the top),
so the pure-torch functions are lifted out of the file by name with ``ast`` and executed as
they stand:
  * get_torch_ref + _gateup_activation_ref   (tests/contrib/moe/test_moe.py)
  * moe_sorting_ref                          (src/contrib/fused_moe.py)
Inputs come from pyhip_b200.synth (seeded); every input tensor is stored beside the outputs
so the fixtures do not depend on the random generator of a later torch version.
"""
import ast
import pathlib
import sys

import numpy as np
import torch

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from pyhip_b200 import quant, synth  # noqa: E402


def lift(path: pathlib.Path, names):
    tree = ast.parse(path.read_text())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in body} == set(names), f"missing functions in {path}"
    ns = {"torch": torch}
    exec(compile(ast.Module(body=body, type_ignores=[]), str(path), "exec"), ns)
    return ns


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str):
    ref = pathlib.Path(ref_root)
    out_dir = pathlib.Path(__file__).resolve().parent
    layer = lift(ref / "tests/contrib/moe/test_moe.py", ["get_torch_ref", "_gateup_activation_ref"])
    sorter = lift(ref / "src/contrib/fused_moe.py", ["moe_sorting_ref"])

    # ---- end-to-end layer, small MXFP4 case and a swiglu variant -------------------------
    T, H, I, E, K = 16, 256, 128, 4, 2
    x = synth.make_hidden(T, H, seed=3)
    tw, ids = synth.make_routing(T, E, K, "softmax", seed=3)
    w1_q, w1_s, w2_q, w2_s = synth.make_weights_mxfp4(E, H, I, seed=3)
    w1 = quant.dequantize_mxfp4(w1_q, w1_s)
    w2 = quant.dequantize_mxfp4(w2_q, w2_s)
    y_silu = layer["get_torch_ref"](x, w1, w2, tw, ids)
    y_swiglu = layer["get_torch_ref"](x, w1, w2, tw, ids, activation="swiglu", swiglu_limit=7.0)
    np.savez_compressed(
        out_dir / "layer_mxfp4_small.npz",
        x=bf16_bits(x), topk_weight=tw.numpy(), topk_ids=ids.numpy(),
        w1_q=w1_q.numpy(), w1_s=w1_s.numpy(), w2_q=w2_q.numpy(), w2_s=w2_s.numpy(),
        w1_deq=bf16_bits(w1), w2_deq=bf16_bits(w2),
        y_silu=bf16_bits(y_silu), y_swiglu=bf16_bits(y_swiglu))

    # ---- FP8 128x128 case -----------------------------------------------------------------
    T, H, I, E, K = 8, 256, 128, 4, 2
    x = synth.make_hidden(T, H, seed=5)
    tw, ids = synth.make_routing(T, E, K, "sigmoid", seed=5)
    w1_q, w1_s, w2_q, w2_s = synth.make_weights_fp8(E, H, I, seed=5)
    w1 = quant.dequantize_fp8_128x128(w1_q, w1_s)
    w2 = quant.dequantize_fp8_128x128(w2_q, w2_s)
    y = layer["get_torch_ref"](x, w1, w2, tw, ids)
    np.savez_compressed(
        out_dir / "layer_fp8_small.npz",
        x=bf16_bits(x), topk_weight=tw.numpy(), topk_ids=ids.numpy(),
        w1_q=w1_q.view(torch.uint8).numpy(), w1_s=w1_s.numpy(),
        w2_q=w2_q.view(torch.uint8).numpy(), w2_s=w2_s.numpy(), y=bf16_bits(y))

    # ---- sorting: the reference function pads to a literal 256, so pin it at B=256 ---------
    T, E, K, B = 300, 16, 4, 256
    tw, ids = synth.make_routing(T, E, K, "zipf", seed=7)
    s_ids, s_w, s_e, nv, _ = sorter["moe_sorting_ref"](ids, tw, E, 8, torch.bfloat16, B)
    n = int(nv[0])
    np.savez_compressed(
        out_dir / "sorting_b256.npz",
        topk_ids=ids.numpy(), topk_weight=tw.numpy(), E=E, B=B,
        sorted_ids=s_ids[:n].numpy().astype(np.uint32), sorted_weights=s_w[:n].numpy(),
        sorted_expert_ids=s_e[: n // B].numpy().astype(np.int32), num_valid=n)
    print("wrote", sorted(p.name for p in out_dir.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of tingqli/pyhip>")
    main(sys.argv[1])
