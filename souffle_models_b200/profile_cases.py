"""Small fixed workloads of the in-scope models, one per invocation: the targets of `ncu` captures.

The reference profiles each model by running it under Nsight Compute and summing per-kernel figures
(python/models/run_ncu_bert.sh:1-8, run_ncu_lstm.sh, run_ncu_swin_trans.sh; the totals land in
python/models/tee:1-2).  The counterpart here:

    ncu --metrics gpu__time_duration.sum,dram__bytes_read.sum --clock-control none --csv --log-file case.csv \\
        python -m souffle_models_b200.profile_cases <case>
    python -m souffle_models_b200.ncu_tables case.csv souffle_

Every case builds its plan on seeded random parameters, makes 3 warm-up calls and 5 timed ones (CUDA events) and
prints the mean time per call.  Cases: bert_layer (1 x 128, one layer), bert_base (1 x 128, 12 layers), bert_layer_b64 (64 x 128
with ragged lengths, one layer), bert_layer_b64_pairs (the same on CTA pairs, desc.pair_mma; set SOUFFLE_PAIR_COOPERATIVE=0
under Nsight Compute, which cannot capture a launch that is both clustered and cooperative), bert_base_b<n> (12 layers
at n sequences, e.g. bert_base_b64, _b32, _b16, _b8: one GPU's share of the benchmark step on 1, 2, 4 and 8 GPUs),
gemm_fc1 (one 8192 x 3072 x 768 product through the plan-less GEMM entry: main loop and plain fp16 epilogue alone),
bert_layer_s384
(the reference's native shape and numerical variant through the blocking drop-in entry, which also returns the five
intermediate tensors), bert_layer_s384_plan (the same launch called back to back), lstm (10 x 256, 100 steps), swin_mlp (256 x 512 x 2048),
swin_pair (14 x 14 x 512, shifts 0 and 3), swin_stage (18 blocks + patch merging), se_module (the reference's ten
shapes, one call each per round).
"""
import sys

import torch

from . import bert, efficientnet, lstm, swin

SE_SHAPES = [(112, 32, 8), (56, 96, 4), (56, 144, 6), (28, 144, 6), (28, 240, 10), (14, 240, 10), (14, 480, 20),
             (14, 672, 28), (7, 672, 28), (7, 1152, 48)]      # (height = width, channels, reduce channels)


def _g(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def _h(shape, g, std=1.0) -> torch.Tensor:
    return (torch.randn(*shape, generator=g) * std).half().cuda()


def _bert_layers(n: int, hidden: int, ffn: int, g, vectors: bool):
    layers = []
    for _ in range(n):
        w = dict(qkv_w=_h((3, hidden, hidden), g, 0.02), proj_w=_h((hidden, hidden), g, 0.02),
                 fc1_w=_h((hidden, ffn), g, 0.02), fc2_w=_h((ffn, hidden), g, 0.02))
        if vectors:
            w.update(qkv_b=_h((3 * hidden,), g, 0.02), proj_b=_h((hidden,), g, 0.02), fc1_b=_h((ffn,), g, 0.02),
                     fc2_b=_h((hidden,), g, 0.02), ln1_g=torch.ones(hidden).half().cuda(), ln1_b=torch.zeros(hidden).half().cuda(),
                     ln2_g=torch.ones(hidden).half().cuda(), ln2_b=torch.zeros(hidden).half().cuda())
        layers.append(w)
    return layers


def _swin_block_params(dim: int, heads: int, window: int, ratio: int, g):
    F, tbl = dim * ratio, (2 * window - 1) ** 2
    one, zero = torch.ones(dim).half().cuda(), torch.zeros(dim).half().cuda()
    return dict(ln1_g=one, ln1_b=zero, qkv_w=_h((dim, 3 * dim), g, 0.02), qkv_b=_h((3 * dim,), g, 0.02),
                rel_bias=_h((tbl, heads), g, 0.02), proj_w=_h((dim, dim), g, 0.02), proj_b=_h((dim,), g, 0.02),
                ln2_g=one, ln2_b=zero, fc1_w=_h((dim, F), g, 0.02), fc1_b=_h((F,), g, 0.02), fc2_w=_h((F, dim), g, 0.02),
                fc2_b=_h((dim,), g, 0.02))


def make_case(name: str):
    """Returns (call, check): `call()` runs the workload once, asynchronously; `check()` raises on a device-side error."""
    g = _g(1234)
    if name in ("bert_layer", "bert_base"):
        n = 1 if name == "bert_layer" else 12
        enc = bert.BertEncoder(1, 128, 12, 64, 3072, _bert_layers(n, 768, 3072, g, True))
        x = _h((1, 128, 768), g)
        y = torch.empty_like(x)
        return (lambda: enc.forward(x, None, y)), enc.status
    if name == "gemm_fc1":
        a, w = _h((8192, 768), g), _h((768, 3072), g, 0.02)
        return (lambda: swin.gemm(a, w, check=False)), (lambda: None)
    if name in ("bert_layer_b64", "bert_layer_b64_pairs") or (name.startswith("bert_base_b") and name[11:].isdigit()):
        n = 1 if name.startswith("bert_layer") else 12
        batch = int(name[11:]) if name.startswith("bert_base_b") else 64
        tuning = dict(pair_mma=1) if name.endswith("_pairs") else None
        enc = bert.BertEncoder(batch, 128, 12, 64, 3072, _bert_layers(n, 768, 3072, g, True), tuning=tuning)
        x = _h((batch, 128, 768), g)
        lens = torch.randint(32, 129, (batch,), generator=g).to(torch.int32).cuda()
        y = torch.empty_like(x)
        return (lambda: enc.forward(x, lens, y)), enc.status
    if name == "bert_layer_s384":
        w = _bert_layers(1, 768, 3072, g, False)[0]
        x = _h((1, 384, 768), g)
        return (lambda: bert.souffle_bert_layer(x, w["qkv_w"], w["proj_w"], w["fc1_w"], w["fc2_w"], 4)), (lambda: None)
    if name == "bert_layer_s384_plan":         # the launch behind the drop-in entry alone: no blocking, no copies out
        w = _bert_layers(1, 768, 3072, g, False)[0]
        enc = bert.BertEncoder(1, 384, 12, 64, 3072, [w], variant=bert.REF_COMPAT, keep_probs=True)
        x = _h((1, 384, 768), g)
        y = torch.empty_like(x)
        return (lambda: enc.forward(x, None, y)), enc.status
    if name == "lstm":
        w_in = ((torch.rand(40, 256, 256, generator=g) - 0.5) / 8).cuda()
        w_st = ((torch.rand(40, 256, 256, generator=g) - 0.5) / 8).cuda()
        x = torch.randn(1, 100, 256, generator=g).cuda()
        plan = lstm.LstmStack(w_in, w_st, 100)
        return (lambda: plan.forward(x)), plan.status
    if name == "swin_mlp":
        src, w1, w2 = _h((256, 512), g), _h((512, 2048), g, 0.02), _h((2048, 512), g, 0.02)
        return (lambda: swin.swin_fused_feed_mlp(src, w1, w2, check=False)), (lambda: None)
    if name in ("swin_pair", "swin_stage"):
        n = 2 if name == "swin_pair" else 18
        blocks = [_swin_block_params(512, 16, 7, 4, g) for _ in range(n)]
        merge = None
        if name == "swin_stage":
            merge = dict(norm_g=torch.ones(2048).half().cuda(), norm_b=torch.zeros(2048).half().cuda(),
                         reduction_w=_h((2048, 1024), g, 0.02))
        plan = swin.SwinBlock(1, 14, 512, 16, 7, 0, blocks, shift_alt=3, merge=merge)
        x = _h((196, 512), g)
        return (lambda: plan.forward(x)), plan.status
    if name == "se_module":
        cases = [(torch.randn(1, c, hw, hw, generator=g).cuda(), (torch.randn(r, c, generator=g) * 0.1).cuda(),
                  (torch.randn(c, r, generator=g) * 0.1).cuda()) for hw, c, r in SE_SHAPES]

        def call():
            for x, wr, we in cases:
                efficientnet.se_module(x, wr, we, check=False)
        return call, (lambda: None)
    raise SystemExit(f"unknown case {name!r}; see the module docstring")


def run(name: str, warmup: int = 3, iters: int = 5) -> float:
    if not torch.cuda.is_available():
        raise SystemExit("profile_cases needs a CUDA device")
    call, check = make_case(name)
    for _ in range(warmup):
        call()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        call()
    e1.record()
    e1.synchronize()
    check()
    us = e0.elapsed_time(e1) * 1000.0 / iters
    print(f"{name}: {us:.1f} us per call")
    return us


if __name__ == "__main__":
    if len(sys.argv) < 2:
        print(__doc__)
        sys.exit(2)
    for case in sys.argv[1:]:
        run(case)
