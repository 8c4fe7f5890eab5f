"""GPU tier: known-answer probes of the two hardware data paths the GEMM main loop relies on --
the copy engine's FP4 unpacking into 128-byte-swizzled shared memory, and the shared->tensor
memory scale copy."""
import ctypes
import os
import pathlib

import numpy as np
import pytest
import torch

from pyhip_b200 import _lib

pytestmark = pytest.mark.gpu
DUMP = os.environ.get("B200MOE_PROBE_DUMP")      # directory to save the probe images in (unset: nothing is written)


def _dump(name, arr):
    if DUMP:
        pathlib.Path(DUMP).mkdir(parents=True, exist_ok=True)
        np.save(pathlib.Path(DUMP) / name, arr)


def _probe(which, inp: torch.Tensor, out_words: int):
    out = torch.zeros(out_words, dtype=torch.int32, device="cuda:0")
    _lib.check(_lib.lib().b200moe_debug_probe(which, ctypes.c_void_p(inp.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "probe")
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_tma_fp4_unpack_image():
    g = torch.Generator().manual_seed(0)
    src = torch.randint(0, 256, (128, 128), dtype=torch.uint8, generator=g)
    raw = _probe(1, src.cuda(), 4096 + 1)
    assert raw[4096] == 0, "TMA wait ran out"
    img = raw[:4096].view(np.uint8).reshape(128, 128)
    _dump("probe_tma_fp4_image.npy", img)
    s = src.numpy()
    for r in range(128):
        for c in range(8):                       # logical 16-byte chunk -> 128-byte-swizzled position
            phys = (c ^ (r & 7)) * 16
            assert np.array_equal(img[r, phys:phys + 16], s[r, c * 16:c * 16 + 16]), (r, c)


def test_scale_copy_to_tensor_memory_layout():
    src = (torch.arange(512, dtype=torch.int64) % 251).to(torch.uint8)
    raw = _probe(2, src.cuda(), 512 + 1)
    assert raw[512] == 0, "tcgen05.cp wait ran out"
    got = raw[:512].astype(np.uint32).reshape(128, 4)
    _dump("probe_utccp.npy", got)
    words = src.numpy().view(np.uint32).reshape(32, 4)       # 32 rows x 16 bytes
    for lane in range(128):
        assert np.array_equal(got[lane], words[lane % 32]), lane


@pytest.mark.parametrize("kind,n", [(0, 256), (1, 256)])
def test_mma_rate_probe_completes(kind, n):
    """The whole-chip dense MMA rate probe the benchmark uses for its tensor roofline (FP4 and FP8 kinds):
    every SM reports, no bounded wait runs out, and the issue loop took a plausible number of cycles."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    count = 2000
    cfg = torch.tensor([kind, n, count, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda:0")
    raw = _probe(4, cfg, sms * 3).reshape(sms, 3)
    assert (raw[:, 2] == 0).all(), "a wait ran out"
    assert (raw[:, 1] > count * 32).all() and (raw[:, 1] < count * 4000).all()


def test_a_wait_that_runs_out_reports_and_leaves_the_context_usable():
    """Failure detection on the device without a fault: a barrier that nothing ever arrives on, a 3 ms limit.  The wait
    gives up, the kernel writes the wait's id into its status word and returns; the next launch on the same context
    works.  This is the path every role of the GEMM kernels takes when a wait runs out (their limit is two seconds)."""
    cfg = torch.tensor([3000], dtype=torch.int32, device="cuda:0")
    raw = _probe(5, cfg, 4)
    assert raw[0] == 0xBEEF and raw[1] == 0
    assert 3000 <= raw[2] < 500000, raw[2]
    test_scale_copy_to_tensor_memory_layout()          # the context is alive and the library still works
