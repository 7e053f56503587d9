"""Generates tests/golden/bert_torch_ref.npz by running the reference's own torch modules
(python/models/bert/bert_torch.py: AttentionModule :17-56, FeedForward :88-104) on CPU in fp32.

Run where the reference checkout is available:
    python tests/golden/make_bert_torch_golden.py /path/to/reference

The reference's attention module calls `.cuda()` on its scale tensor (bert_torch.py:46);
on a CPU-only host that call is made a no-op for the duration of this script.  Nothing of
the reference is copied: only its inputs, parameters and outputs are stored.
"""
import contextlib
import io
import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "python", "models", "bert"))
    import bert_torch  # the reference module

    torch.Tensor.cuda = lambda self, *a, **k: self       # CPU-only host
    torch.manual_seed(20240611)
    B, S, heads, hd, ffn = 1, 16, 2, 32, 256
    H = heads * hd
    cpu = torch.device("cpu")
    attn = bert_torch.AttentionModule(B, S, heads, hd, device=cpu, dtype=torch.float32, fused_qkv=False)
    ff = bert_torch.FeedForward(H, ffn, device=cpu, dtype=torch.float32)
    x = torch.randn(B, S, H)
    with torch.no_grad(), contextlib.redirect_stdout(io.StringIO()):
        ln1 = attn(x)
        out = ff(ln1)
    t = lambda lin: lin.weight.detach().t().contiguous().numpy()      # -> [K][N]
    b = lambda lin: lin.bias.detach().numpy()
    np.savez_compressed(
        os.path.join(os.path.dirname(os.path.abspath(__file__)), "bert_torch_ref.npz"),
        shape=np.array([B, S, heads, hd, ffn]), x=x.numpy(),
        qkv_w=np.stack([t(attn.query), t(attn.key), t(attn.value)]),
        qkv_b=np.stack([b(attn.query), b(attn.key), b(attn.value)]),
        proj_w=t(attn.fc), proj_b=b(attn.fc),
        fc1_w=t(ff.linear1), fc1_b=b(ff.linear1), fc2_w=t(ff.linear2), fc2_b=b(ff.linear2),
        ln2_g=ff.norm2.weight.detach().numpy(), ln2_b=ff.norm2.bias.detach().numpy(),
        ln1=ln1.numpy().reshape(B * S, H), out=out.numpy().reshape(B * S, H),
        # the reference divides the scores by head size, not its square root (bert_torch.py:46-47)
        scale=np.array([1.0 / hd]), eps=np.array([1e-5]))


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("SOUFFLE_REFERENCE"):
        raise SystemExit("usage: make_bert_torch_golden.py <reference checkout>   (or set SOUFFLE_REFERENCE)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["SOUFFLE_REFERENCE"])
