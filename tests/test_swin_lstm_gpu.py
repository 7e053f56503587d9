"""Parity of the GEMM / Swin MLP / LSTM entry points (through the C ABI) with the oracle."""
import os

import pytest
import torch

from oracle import souffle_oracle as so

pytestmark = pytest.mark.gpu


def _report(name, value):
    """Measured parity figures: printed (pytest -s) and appended to $SOUFFLE_PARITY_LOG when that is set."""
    line = f"{name} = {value:.3e}"
    print(line)
    path = os.environ.get("SOUFFLE_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")


def _rand(shape, seed, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).half()


@pytest.mark.parametrize("M,N,K", [(256, 2048, 512), (256, 512, 2048), (128, 64, 64), (200, 256, 128), (1, 64, 64)])
def test_gemm_matches_oracle(M, N, K):
    from souffle_models_b200 import swin
    a, w = _rand((M, K), 1), _rand((K, N), 2, 0.05)
    c = swin.swin_ffn(a.cuda(), w.cuda(), M, N, K)
    want = so.gemm_kn(a, w)
    assert (c.float().cpu() - want).abs().max() < 2e-3 * max(1.0, want.abs().max().item())


def test_swin_fused_mlp_and_fc2():
    from souffle_models_b200 import swin
    src, w1, w2 = _rand((256, 512), 3), _rand((512, 2048), 4, 0.02), _rand((2048, 512), 5, 0.02)
    hidden, out = swin.swin_fused_feed_mlp(src.cuda(), w1.cuda(), w2.cuda())
    h1, o1 = so.swin_mlp(src, w1, w2, emulate_fp16=True)
    assert (hidden.float().cpu() - h1).abs().max() < 2e-3
    assert (out.float().cpu() - o1).abs().max() < 4e-3
    y = swin.swin_trans_fc2(hidden.reshape(1, 256, 2048), w2.cuda())
    assert y.shape == (1, 256, 512) and (y.float().cpu().reshape(256, 512) - o1).abs().max() < 4e-3
    assert swin.bench_swin_ffn(256, 2048, 512, 2, 5, 2) > 0


@pytest.mark.parametrize("layers,hidden,steps", [(3, 64, 8), (10, 256, 100), (2, 128, 5)])
def test_lstm_matches_oracle(layers, hidden, steps):
    """Hidden states within 5e-3 (the stated bar) and, because that bar is loose for values this
    small, also within 2e-5 + 1e-3 relative."""
    from souffle_models_b200 import lstm
    x, w_in, w_st = so.make_lstm_params(layers, hidden, steps, seed=1237)
    for delay in (False, True):
        plan = lstm.LstmStack(w_in.cuda(), w_st.cuda(), steps, ref_input_delay=delay)
        y = plan.forward(x.float().cuda())
        plan.status()
        want = so.lstm_forward(x, w_in, w_st, ref_input_delay=delay)
        err = (y.cpu() - want).abs()
        assert err.max() < 5e-3
        assert (err <= 2e-5 + 1e-3 * want.abs()).all()
        y2 = plan.forward(x.float().cuda())
        plan.status()
        assert torch.equal(y, y2)


def test_lstm_larger_weights_and_bias():
    """Weights large enough that the state does not vanish through the stack."""
    from souffle_models_b200 import lstm
    g = torch.Generator().manual_seed(9)
    L, H, T = 4, 256, 20
    w_in = ((torch.rand(4 * L, H, H, generator=g) - 0.5) * 0.5).half()
    w_st = ((torch.rand(4 * L, H, H, generator=g) - 0.5) * 0.5).half()
    bias = torch.randn(L, H, generator=g) * 0.1
    x = torch.randn(1, T, H, generator=g).half()
    plan = lstm.LstmStack(w_in.cuda(), w_st.cuda(), T, bias=bias.cuda())
    y = plan.forward(x.float().cuda())
    plan.status()
    want = so.lstm_forward(x, w_in, w_st, bias=bias)
    assert want.abs().max() > 0.1
    assert (y.cpu() - want).abs().max() < 5e-3


def test_fused_lstm_drop_in_signature():
    from souffle_models_b200 import lstm
    x, w_in, w_st = so.make_lstm_params()
    y = lstm.fused_lstm(x.float().cuda(), w_in.float().cuda(), w_st.float().cuda())
    assert y.shape == (1, 100, 256) and y.dtype == torch.float32
    assert (y.cpu() - so.lstm_forward(x, w_in, w_st, ref_input_delay=True)).abs().max() < 5e-3


def test_fused_lstm_with_weights_fp16_cannot_represent():
    """The drop-in entry takes the reference's fp32 weights and keeps them as fp16 on the device
    (cpp/lstm/lstm_binding.cu:30-37 multiplies in fp32): with weights that are NOT fp16-valued the rounding of the
    weights is part of the error.  Measured against the fp32 oracle on the unrounded weights."""
    from souffle_models_b200 import lstm
    g = torch.Generator().manual_seed(77)
    w_in = (torch.rand(40, 256, 256, generator=g) - 0.5) / 8.0          # fp32, not rounded to fp16
    w_st = (torch.rand(40, 256, 256, generator=g) - 0.5) / 8.0
    x = torch.randn(1, 100, 256, generator=g)
    assert not torch.equal(w_in, w_in.half().float())
    y = lstm.fused_lstm(x.cuda(), w_in.cuda(), w_st.cuda())
    want = so.lstm_forward(x, w_in, w_st, ref_input_delay=True)
    err = (y.cpu() - want).abs()
    _report("LSTM 10 x 256 x 100 with fp32 weights stored as fp16: max-abs on hidden states", err.max().item())
    _report("LSTM 10 x 256 x 100 with fp32 weights stored as fp16: largest |h|", want.abs().max().item())
    assert err.max() < 5e-3


@pytest.mark.parametrize("P,M,N", [(1, 300, 768), (3, 64, 512), (2, 1000, 1024), (1, 5, 128)])
def test_layernorm_entry_point(P, M, N):
    from souffle_models_b200 import swin
    g = torch.Generator().manual_seed(4)
    part = torch.randn(P, M, N, generator=g)
    resid, bias = _rand((M, N), 5), _rand((N,), 6, 0.1)
    gamma, beta = (1 + torch.randn(N, generator=g) * 0.1).half(), _rand((N,), 7, 0.1)
    out = swin.layernorm(part.cuda(), resid.cuda(), bias.cuda(), gamma.cuda(), beta.cuda(), eps=1e-12)
    want = so.layer_norm(part.sum(0) + bias.float() + resid.float(), gamma, beta, 1e-12)
    assert (out.float().cpu() - want).abs().max() < 5e-3


@pytest.mark.parametrize("shift", [0, 3])
def test_swin_block_matches_oracle(shift):
    """Benchmark config 4: 14x14 tokens, C=512, 16 heads x 32, window 7, shifted pair, bias table, GELU MLP."""
    from souffle_models_b200 import swin
    cfg = so.SwinConfig()
    p = so.make_swin_params(cfg, 1238 + shift, zero_bias=False)
    x = _rand((196, 512), 11 + shift)
    blk = swin.SwinBlock(1, 14, 512, 16, 7, shift, {k: v.cuda() for k, v in p.items()})
    y = blk.forward(x.cuda())
    blk.status()
    want = so.swin_block(cfg, x, p, shift)
    err = (y.float().cpu() - want).abs()
    e16 = (y.float().cpu() - so.swin_block(cfg, x, p, shift, emulate_fp16=True)).abs().max().item()
    _report(f"Swin block shift {shift}: max-abs vs fp32 oracle", err.max().item())
    _report(f"Swin block shift {shift}: max-abs vs fp16-storage oracle", e16)
    # the block's output is the un-normalised residual stream (|y| up to ~6, fp16 ulp 4e-3 there); measured 3e-3
    assert e16 < 1e-2
    assert err.max() < 1e-2 and err.pow(2).mean().sqrt() < 2e-3
    y2 = blk.forward(x.cuda())
    blk.status()
    assert torch.equal(y, y2)


def test_swin_shifted_pair_as_one_launch():
    """Benchmark config 4 as it is stated: the pair of blocks (shift 0, then shift 3), chained inside one launch."""
    from souffle_models_b200 import swin
    cfg = so.SwinConfig()
    ps = [so.make_swin_params(cfg, 300 + i, zero_bias=False) for i in range(2)]
    x = _rand((196, 512), 31)
    pair = swin.SwinBlock(1, 14, 512, 16, 7, 0, [{k: v.cuda() for k, v in p.items()} for p in ps], shift_alt=3)
    y = pair.forward(x.cuda())
    pair.status()
    mid = so.swin_block(cfg, x, ps[0], 0)
    want = so.swin_block(cfg, mid.half().float(), ps[1], 3)       # the block boundary is an fp16 tensor on the GPU
    err = (y.float().cpu() - want).abs()
    _report("Swin shifted pair: max-abs vs fp32 oracle", err.max().item())
    assert err.max() < 1.5e-2 and err.pow(2).mean().sqrt() < 2e-3


def test_swin_block_batch2_window8():
    from souffle_models_b200 import swin
    cfg = so.SwinConfig(res=16, dim=256, heads=8, window=8)
    p = so.make_swin_params(cfg, 77, zero_bias=False)
    x = _rand((2 * 256, 256), 5)
    blk = swin.SwinBlock(2, 16, 256, 8, 8, 4, {k: v.cuda() for k, v in p.items()})
    y = blk.forward(x.cuda())
    blk.status()
    want = torch.cat([so.swin_block(cfg, x[:256], p, 4), so.swin_block(cfg, x[256:], p, 4)])
    _report("Swin block batch 2, window 8: max-abs vs fp32 oracle", (y.float().cpu() - want).abs().max().item())
    assert (y.float().cpu() - want).abs().max() < 1e-2


@pytest.mark.parametrize("batch,res,dim,heads,window", [(1, 14, 512, 16, 7), (2, 16, 256, 8, 8), (3, 14, 128, 4, 7)])
def test_swin_stage_with_patch_merging(batch, res, dim, heads, window):
    """A block followed by the patch merging that ends a stage, in one launch: 4*dim = 2048 (the wide-row LayerNorm),
    1024 and 512; several images, so the gather crosses image boundaries."""
    from souffle_models_b200 import swin
    cfg = so.SwinConfig(res=res, dim=dim, heads=heads, window=window)
    p = so.make_swin_params(cfg, 500 + dim, zero_bias=False)
    m = so.make_swin_merge_params(cfg, 600 + dim, zero_bias=False)
    T = res * res
    x = _rand((batch * T, dim), 41)
    shift = window // 2
    plan = swin.SwinBlock(batch, res, dim, heads, window, shift, {k: v.cuda() for k, v in p.items()},
                          merge={k: v.cuda() for k, v in m.items()})
    y = plan.forward(x.cuda())
    plan.status()
    assert y.shape == (batch * (res // 2) ** 2, 2 * dim)
    want = torch.cat([so.swin_patch_merge(cfg, so.swin_block(cfg, x[i * T:(i + 1) * T], p, shift).half().float(), m)
                      for i in range(batch)])
    err = (y.float().cpu() - want).abs()
    _report(f"Swin block + patch merging, dim {dim}: max-abs vs fp32 oracle", err.max().item())
    assert err.max() < 1.5e-2 and err.pow(2).mean().sqrt() < 3e-3
    y2 = plan.forward(x.cuda())
    plan.status()
    assert torch.equal(y, y2)


def test_swin_stage3_eighteen_blocks_and_merge():
    """The whole stage 3 of Swin-B as one launch: 18 blocks (shifts 0, 3, 0, ...) and the patch merging after them,
    against 18 chained oracle blocks (the block boundary is an fp16 tensor on the GPU) and the oracle's merge."""
    from souffle_models_b200 import swin
    cfg = so.SwinConfig()
    ps = [so.make_swin_params(cfg, 900 + i, zero_bias=False) for i in range(18)]
    m = so.make_swin_merge_params(cfg, 950, zero_bias=False)
    x = _rand((196, 512), 47)
    y = swin.swin_stage(x.cuda(), [{k: v.cuda() for k, v in p.items()} for p in ps], {k: v.cuda() for k, v in m.items()})
    assert y.shape == (49, 1024)
    cur32, cur16 = x.float(), x.float()
    for i, p in enumerate(ps):
        shift = 3 if i % 2 else 0
        cur32 = so.swin_block(cfg, cur32, p, shift).half().float()
        cur16 = so.swin_block(cfg, cur16, p, shift, emulate_fp16=True).half().float()
    want32, want16 = so.swin_patch_merge(cfg, cur32, m), so.swin_patch_merge(cfg, cur16, m)
    got = y.float().cpu()
    e32, e16 = (got - want32).abs(), (got - want16).abs()
    _report("Swin stage 3 (18 blocks + merge): max-abs vs fp32 oracle", e32.max().item())
    _report("Swin stage 3 (18 blocks + merge): max-abs vs fp16-storage oracle", e16.max().item())
    _report("Swin stage 3 (18 blocks + merge): rms vs fp32 oracle", e32.pow(2).mean().sqrt().item())
    assert torch.isfinite(got).all()
    assert e32.max() < 1.5e-2 and e32.pow(2).mean().sqrt() < 3e-3          # measured 5.8e-3 / 1.4e-3
    assert e16.max() < 1.5e-2                                               # measured 5.2e-3


def test_swin_stage_entry_and_merge_shape_errors():
    from souffle_models_b200 import swin
    cfg = so.SwinConfig()
    ps = [so.make_swin_params(cfg, 700 + i) for i in range(2)]
    m = so.make_swin_merge_params(cfg, 710)
    x = _rand((196, 512), 43)
    y = swin.swin_stage(x.cuda(), [{k: v.cuda() for k, v in p.items()} for p in ps], {k: v.cuda() for k, v in m.items()})
    mid = so.swin_block(cfg, so.swin_block(cfg, x, ps[0], 0).half().float(), ps[1], 3)
    want = so.swin_patch_merge(cfg, mid.half().float(), m)
    assert y.shape == (49, 1024) and (y.float().cpu() - want).abs().max() < 1.5e-2
    big = so.SwinConfig(dim=768, heads=24)
    with pytest.raises(RuntimeError, match="patch merging"):
        swin.SwinBlock(1, 14, 768, 24, 7, 0, {k: v.cuda() for k, v in so.make_swin_params(big, 1).items()},
                       merge={k: v.cuda() for k, v in so.make_swin_merge_params(big, 2).items()})


def test_lstm_and_swin_mlp_match_reference_cuda_outputs(golden_dir):
    """This library against what the reference's own kernels produced on a B200 (tests/golden/ref_cuda_lstm_swin.npz):
    the LSTM in the reference's feeding order, and the fused MLP on its seeded inputs."""
    import numpy as np
    from souffle_models_b200 import lstm, swin
    g = np.load(f"{golden_dir}/ref_cuda_lstm_swin.npz")
    x, w_in, w_st = so.make_lstm_params()
    plan = lstm.LstmStack(w_in.cuda(), w_st.cuda(), 100, ref_input_delay=True)
    y = plan.forward(x.float().cuda())
    plan.status()
    want = torch.from_numpy(g["lstm_y"])
    err = (y.cpu()[0] - want).abs()
    assert err.max() < 5e-3 and (err <= 2e-5 + 1e-3 * want.abs()).all()
    gen = torch.Generator().manual_seed(1238)
    src = torch.randn(256, 512, generator=gen).half()
    w1, w2 = (torch.randn(512, 2048, generator=gen) * 0.02).half(), (torch.randn(2048, 512, generator=gen) * 0.02).half()
    hidden, out = swin.swin_fused_feed_mlp(src.cuda(), w1.cuda(), w2.cuda())
    assert (hidden[:32].float().cpu() - torch.from_numpy(g["swin_hidden_head"]).float()).abs().max() < 1e-2
    assert (out.float().cpu() - torch.from_numpy(g["swin_out"]).float()).abs().max() < 1.5e-2


def test_lstm_launch_mode_and_profile_case():
    """The default launch form carries the cluster dimension alone (mode 0); the small fixed workload used for ncu
    captures runs and reports a time."""
    from souffle_models_b200 import _lib, profile_cases
    assert profile_cases.run("lstm", warmup=1, iters=2) > 0
    assert _lib.load().souffle_lstm_launch_mode() in (0, 1)
