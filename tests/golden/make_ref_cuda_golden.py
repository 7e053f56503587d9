"""Generates tests/golden/ref_cuda_bert_s384.npz and ref_cuda_lstm_swin.npz from the reference's own CUDA kernels,
and prints their kernel times (CUDA events inside the harness, mean of 30 launches).

Needs a B200 and oracle/_ref/libsouffle_ref.so (built by `make -C oracle ref REF=<reference>` from
the reference sources: fused_sqq_bert_attn + fused_sqq_feedforward_pipelined_v2, launched as
cpp/bert/bert_binding.cu:395-528 does at opt_level 4, shape [1,384,768]).
    python tests/golden/make_ref_cuda_golden.py [out.npz]
Inputs are the seeded tensors of oracle.souffle_oracle (seed 1234); the file keeps the first 48
rows of each of the six stage outputs and (sum, abs-sum) of the whole tensors.
The second file holds the output of the LSTM wavefront kernel (lstm_reuse_shared_memory_v10_vec<1,10,256,100>,
launched as cpp/lstm/lstm_binding.cu:44-70 does) on make_lstm_params() and of the fused Swin MLP
(swin_transformer_fused_fc1_fc2, cpp/swin_transformer/swin_transformer_binding.cu:155-209) on seed 1238.
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
    for opt in (3, 4):
        rc = ref.ref_bert_layer_s384(P(x), P(w["qkv_w"]), P(w["proj_w"]), P(w["fc1_w"]), P(w["fc2_w"]), opt,
                                     *[P(outs[k]) for k in ("qkv", "probs", "ctx", "ln1", "fc1", "out")], 30, C.byref(us))
        torch.cuda.synchronize()
        print(f"reference BERT layer, seq 384, opt_level {opt}: rc {rc}, {us.value:.1f} us (kernels only)")

    gold = {}
    xl, w_in, w_st = so.make_lstm_params()
    y = torch.zeros(1, 100, 256, device="cuda")
    keep = [xl.float().cuda(), w_in.float().cuda(), w_st.float().cuda()]
    rc = ref.ref_lstm_10x256x100(P(keep[0]), P(keep[1]), P(keep[2]), P(y), 30, C.byref(us))
    torch.cuda.synchronize()
    if rc != 0:
        raise SystemExit(f"reference LSTM launch failed with {rc}")
    print(f"reference LSTM 10 x 256, 100 steps: {us.value:.1f} us")
    gold["lstm_y"] = y.cpu().numpy().reshape(100, 256)
    g = torch.Generator().manual_seed(1238)
    src = torch.randn(256, 512, generator=g).half()
    w1, w2 = (torch.randn(512, 2048, generator=g) * 0.02).half(), (torch.randn(2048, 512, generator=g) * 0.02).half()
    hid, o = z(256, 2048), z(256, 512)
    keep = [src.cuda(), w1.cuda(), w2.cuda()]
    rc = ref.ref_swin_mlp_256x512x2048(P(keep[0]), P(keep[1]), P(keep[2]), P(hid), P(o), 30, C.byref(us))
    torch.cuda.synchronize()
    if rc != 0:
        raise SystemExit(f"reference Swin MLP launch failed with {rc}")
    print(f"reference Swin fused MLP 256 x 512 x 2048: {us.value:.1f} us")
    gold["swin_hidden_head"] = hid[:32].cpu().numpy()
    gold["swin_out"] = o.cpu().numpy()
    np.savez_compressed(os.path.join(os.path.dirname(out_path), "ref_cuda_lstm_swin.npz"), **gold)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                            "ref_cuda_bert_s384.npz"))
