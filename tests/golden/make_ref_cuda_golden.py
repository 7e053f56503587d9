"""Generates tests/golden/ref_cuda_bert_s384.npz from the reference's own fused CUDA kernels.

Needs a B200 and oracle/_ref/libsouffle_ref.so (built by `make -C oracle ref REF=<reference>` from
the reference sources: fused_sqq_bert_attn + fused_sqq_feedforward_pipelined_v2, launched as
cpp/bert/bert_binding.cu:395-528 does at opt_level 4, shape [1,384,768]).
    python tests/golden/make_ref_cuda_golden.py [out.npz]
Inputs are the seeded tensors of oracle.souffle_oracle (seed 1234); the file keeps the first 48
rows of each of the six stage outputs and (sum, abs-sum) of the whole tensors.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import souffle_oracle as so  # noqa: E402


def main(out_path: str) -> None:
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libsouffle_ref.so"))
    cfg = so.BertConfig(1, 384, 12, 64, 3072, "ref")
    w = {k: v.cuda() for k, v in so.make_bert_weights(cfg, 1234, 1)[0].items()}
    x = so.make_bert_input(cfg, 1234)[0].cuda()
    z = lambda *s: torch.zeros(*s, dtype=torch.half, device="cuda")
    outs = dict(qkv=z(3, 12, 384, 64), probs=z(12, 384, 384), ctx=z(384, 768), ln1=z(384, 768),
                fc1=z(384, 3072), out=z(384, 768))
    P = lambda t: C.c_void_p(t.data_ptr())
    us = C.c_float()
    rc = ref.ref_bert_layer_s384(P(x), P(w["qkv_w"]), P(w["proj_w"]), P(w["fc1_w"]), P(w["fc2_w"]), 4,
                                 *[P(outs[k]) for k in ("qkv", "probs", "ctx", "ln1", "fc1", "out")], 1,
                                 C.byref(us))
    torch.cuda.synchronize()
    if rc != 0:
        raise SystemExit(f"reference launch failed with {rc}")
    gold = {}
    for k, t in outs.items():
        a = t.float().cpu().reshape(-1, t.shape[-1])
        gold[f"bert_{k}_head"] = a[:48].half().numpy()
        gold[f"bert_{k}_sum"] = np.array([a.double().sum().item(), a.double().abs().sum().item()])
    np.savez_compressed(out_path, **gold)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                            "ref_cuda_bert_s384.npz"))
