"""Generates tests/golden/ref_cuda_se.npz from the reference's own fused squeeze-and-excite kernel
(efficientnet_se_module_v2_short_cut_fused, cpp/efficientnet/kernels/se_module_global_fused.cu:316-444),
and prints its kernel time per shape (CUDA events inside the harness, mean of 30 launches).

Needs a B200 and oracle/_ref/libsouffle_ref.so (built by `make -C oracle ref REF=<reference>`).
    python tests/golden/make_ref_se_golden.py [out.npz]
Shapes: the four of the reference's dispatch table (cpp/efficientnet/efficientnet_se_module_binding.cu:181-208)
that run one channel per block.  Inputs are seeded (seed 7 + channels, the draw order of tests/test_se_gpu.py);
the file keeps the pooled means, the first two and the last channel image of the output, and whole-tensor sums.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

SHAPES = [(56, 96, 4), (28, 144, 6), (14, 240, 10), (14, 480, 20)]      # (height = width, channels, reduce)


def se_case(h: int, c: int, r: int):
    g = torch.Generator().manual_seed(7 + c)
    x = torch.randn(1, c, h, h, generator=g)
    wr = torch.randn(r, c, generator=g) * 0.2
    we = torch.randn(c, r, generator=g) * 0.5
    return x, wr, we


def main(out_path: str) -> None:
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libsouffle_ref.so"))
    P = lambda t: C.c_void_p(t.data_ptr())
    gold = {}
    for h, c, r in SHAPES:
        x, wr, we = se_case(h, c, r)
        xd, wrd, wed = x.cuda(), wr.cuda(), we.cuda()
        pooled, out = torch.zeros(c, device="cuda"), torch.zeros_like(xd)
        us = C.c_float()
        rc = ref.ref_se_module(h, c, r, P(xd), P(wrd), P(wed), P(pooled), P(out), 30, C.byref(us))
        torch.cuda.synchronize()
        if rc != 0:
            raise SystemExit(f"reference SE launch failed with {rc} for shape {(h, c, r)}")
        print(f"reference SE module {c} x {h} x {h}, reduce {r}: {us.value:.1f} us")
        o = out.cpu()[0]
        key = f"se_{h}_{c}_{r}"
        gold[key + "_pooled"] = pooled.cpu().numpy()
        gold[key + "_out_head"] = torch.stack([o[0], o[1], o[c - 1]]).numpy()
        gold[key + "_out_sum"] = np.array([o.double().sum().item(), o.double().abs().sum().item()])
    np.savez_compressed(out_path, **gold)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cuda_se.npz"))
