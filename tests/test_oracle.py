"""CPU checks of the oracle against the golden vectors (no GPU, no native compute)."""
import numpy as np
import pytest
import torch

from oracle import souffle_oracle as so


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_bert_layer_matches_reference_torch_modules(golden_dir):
    """Oracle == the reference's AttentionModule + FeedForward (python/models/bert/bert_torch.py)
    run on CPU fp32; vectors from tests/golden/make_bert_torch_golden.py."""
    g = np.load(f"{golden_dir}/bert_torch_ref.npz")
    B, S, h, d, F = [int(v) for v in g["shape"]]
    cfg = so.BertConfig(B, S, h, d, F, "std")
    w = {k: _t(g[k]) for k in ("qkv_w", "qkv_b", "proj_w", "proj_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b", "ln2_g", "ln2_b")}
    w["ln1_g"], w["ln1_b"] = torch.ones(h * d), torch.zeros(h * d)
    r = so.bert_layer(cfg, _t(g["x"]), w, scale=float(g["scale"][0]), act="relu", eps=float(g["eps"][0]))
    assert (r["ln1"] - _t(g["ln1"])).abs().max() < 1e-5
    assert (r["out"] - _t(g["out"])).abs().max() < 1e-5


def test_ref_compat_matches_reference_cuda_kernels(golden_dir):
    """Oracle (REF_COMPAT) vs outputs of the reference's own fused kernels (fused_sqq_bert_attn +
    fused_sqq_feedforward_pipelined_v2, built for sm_100a by oracle/Makefile and run on a B200;
    stored: first 48 rows of each of the six stage outputs and whole-tensor sums).  The reference
    accumulates in fp16, so the tolerance is its own test's (cpp/bert/test_souffle_bert_layer.py:209-214)."""
    g = np.load(f"{golden_dir}/ref_cuda_bert_s384.npz")
    cfg = so.BertConfig(1, 384, 12, 64, 3072, "ref")
    w = so.make_bert_weights(cfg, 1234, 1)[0]
    x, _ = so.make_bert_input(cfg, 1234)
    r = so.bert_layer(cfg, x, w)
    for k, atol in (("qkv", 1e-2), ("probs", 1e-3), ("ctx", 1e-2), ("ln1", 1e-2), ("fc1", 1e-2), ("out", 2e-2)):
        want = r[k].reshape(-1, r[k].shape[-1])
        got = _t(g[f"bert_{k}_head"]).float()
        assert (got - want[:48]).abs().max() < atol, k
        s, sa = g[f"bert_{k}_sum"]
        assert abs(sa - want.double().abs().sum().item()) / max(1.0, sa) < 2e-3, k


def test_lstm_and_swin_mlp_match_reference_cuda_kernels(golden_dir):
    """Oracle vs outputs of the reference's own kernels run on a B200 (tests/golden/make_ref_cuda_golden.py):
    lstm_reuse_shared_memory_v10_vec<1,10,256,100> on make_lstm_params() -- fp32 throughout, so the restatement with
    the kernel's one-step input delay agrees to rounding, and the un-delayed form does not -- and the fused Swin MLP
    (fp16 accumulation in the reference, hence its own 1e-2 tolerance)."""
    g = np.load(f"{golden_dir}/ref_cuda_lstm_swin.npz")
    x, w_in, w_st = so.make_lstm_params()
    y = _t(g["lstm_y"])
    assert (so.lstm_forward(x, w_in, w_st, ref_input_delay=True)[0] - y).abs().max() < 2e-6
    assert (so.lstm_forward(x, w_in, w_st)[0] - y).abs().max() > 5e-5
    gen = torch.Generator().manual_seed(1238)
    src = torch.randn(256, 512, generator=gen).half()
    w1, w2 = (torch.randn(512, 2048, generator=gen) * 0.02).half(), (torch.randn(2048, 512, generator=gen) * 0.02).half()
    h1, o1 = so.swin_mlp(src, w1, w2, emulate_fp16=True)
    assert (_t(g["swin_hidden_head"]).float() - h1[:32]).abs().max() < 1e-2
    assert (_t(g["swin_out"]).float() - o1).abs().max() < 1.5e-2


def test_gelu_and_layernorm_basics():
    x = torch.linspace(-6, 6, 101)
    assert (so.gelu_tanh(x) - torch.nn.functional.gelu(x, approximate="tanh")).abs().max() < 1e-6
    z = torch.randn(7, 64)
    y = so.layer_norm(z, torch.ones(64), torch.zeros(64), 1e-12)
    assert y.mean(-1).abs().max() < 1e-5 and (y.var(-1, unbiased=False) - 1).abs().max() < 1e-4


def test_length_mask_equals_truncation():
    """Keys past a sequence's length carry the additive -1e4 mask (softmax.cu:22-24): valid query
    rows must equal the result of running the truncated sequence alone."""
    cfg = so.BertConfig(2, 32, 2, 64, 256, "std")
    w = so.make_bert_weights(cfg, 3, 1, zero_bias=False)[0]
    x, _ = so.make_bert_input(cfg, 3)
    lens = torch.tensor([20, 32], dtype=torch.int32)
    full = so.bert_layer(cfg, x, w, lens)["out"].reshape(2, 32, -1)
    short = so.bert_layer(so.BertConfig(1, 20, 2, 64, 256, "std"), x[0:1, :20], w)["out"].reshape(20, -1)
    assert (full[0, :20] - short).abs().max() < 1e-4


def test_stack_is_layer_composition():
    cfg = so.BertConfig(1, 16, 2, 64, 128, "std")
    layers = so.make_bert_weights(cfg, 9, 3)
    x, _ = so.make_bert_input(cfg, 9)
    cur = x.float().reshape(16, -1)
    for w in layers:
        cur = so.bert_layer(cfg, cur, w)["out"]
    assert torch.equal(cur, so.bert_stack(cfg, x, layers))


def test_lstm_cell_semantics_and_reference_feed_order():
    x, w_in, w_st = so.make_lstm_params(layers=3, hidden=64, steps=8, seed=5)
    y = so.lstm_forward(x, w_in, w_st)
    # one cell by hand: gates i, j, f, o; c' = c*sigmoid(f+1) + sigmoid(i)*tanh(j); h' = tanh(c')*sigmoid(o)
    g = (w_in.float()[:4] @ x.float()[0, 0])
    c = torch.sigmoid(g[0]) * torch.tanh(g[1])
    h0 = torch.tanh(c) * torch.sigmoid(g[3])
    g1 = (w_in.float()[4:8] @ h0)
    c1 = torch.sigmoid(g1[0]) * torch.tanh(g1[1])
    h1 = torch.tanh(c1) * torch.sigmoid(g1[3])
    g2 = (w_in.float()[8:12] @ h1)
    c2 = torch.sigmoid(g2[0]) * torch.tanh(g2[1])
    h2 = torch.tanh(c2) * torch.sigmoid(g2[3])
    assert (y[0, 0] - h2).abs().max() < 1e-6
    # the reference kernel consumes x one step late: first output row is the zero-input response
    yd = so.lstm_forward(x, w_in, w_st, ref_input_delay=True)
    assert yd[0, 0].abs().max() == 0
    assert (yd[0, 1:] - so.lstm_forward(x[:, :-1], w_in, w_st)[0]).abs().max() < 1e-6


def test_swin_block_window_algebra():
    cfg = so.SwinConfig()
    idx = so.swin_rel_index(cfg.window)
    assert idx.min() == 0 and idx.max() == (2 * cfg.window - 1) ** 2 - 1 and idx.shape == (49, 49)
    assert torch.equal(idx.diagonal(), torch.full((49,), idx[0, 0]))
    assert so.swin_shift_mask(14, 7, 0).abs().max() == 0
    m = so.swin_shift_mask(14, 7, 3)
    assert m.shape == (4, 49, 49) and m[0].abs().max() == 0 and m[3].min() == -100
    p = so.make_swin_params(cfg, 1238)
    x = torch.randn(196, 512, generator=torch.Generator().manual_seed(1)).half()
    for shift in (0, 3):
        y = so.swin_block(cfg, x, p, shift)
        assert y.shape == (196, 512) and torch.isfinite(y).all()
    # a permutation of tokens inside one window leaves other windows' outputs unchanged (shift 0)
    x2 = x.clone().reshape(14, 14, 512)
    x2[0, 0], x2[1, 1] = x[15].clone(), x[0].clone()
    y0 = so.swin_block(cfg, x, p, 0).reshape(14, 14, 512)
    y2 = so.swin_block(cfg, x2.reshape(196, 512), p, 0).reshape(14, 14, 512)
    assert (y0[7:, :] - y2[7:, :]).abs().max() < 1e-5 and (y0[:7, 7:] - y2[:7, 7:]).abs().max() < 1e-5


def test_swin_mlp_and_gemm():
    g = torch.Generator().manual_seed(2)
    a = torch.randn(8, 64, generator=g).half()
    w1 = torch.randn(64, 128, generator=g).half()
    w2 = torch.randn(128, 64, generator=g).half()
    h, o = so.swin_mlp(a, w1, w2)
    assert torch.allclose(h, a.float() @ w1.float()) and torch.allclose(o, h @ w2.float())


def test_se_module_hand_computed():
    """One channel pair, 2 x 2 image: every number of the squeeze-and-excite chain by hand."""
    import math
    x = torch.tensor([[[[1.0, 2.0], [3.0, 4.0]], [[0.0, 0.0], [0.0, 8.0]]]])       # means 2.5 and 2.0
    wr = torch.tensor([[1.0, -1.0]])                                                 # s = 0.5
    we = torch.tensor([[2.0], [0.0]])
    pooled, out = so.se_module(x, wr, we)
    assert torch.allclose(pooled, torch.tensor([[2.5, 2.0]]))
    r = 0.5 / (1.0 + math.exp(-0.5))
    g0, g1 = 1.0 / (1.0 + math.exp(-2.0 * r)), 0.5
    assert torch.allclose(out[0, 0], x[0, 0] + g0, atol=1e-6) and torch.allclose(out[0, 1], x[0, 1] + g1, atol=1e-6)


def test_se_module_matches_reference_cuda_kernel(golden_dir):
    """Oracle vs outputs of the reference's own fused squeeze-and-excite kernel run on a B200
    (tests/golden/make_ref_se_golden.py; efficientnet_se_module_v2_short_cut_fused, fp32 throughout): the four
    shapes of its dispatch table that run one channel per block."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("make_ref_se_golden", os.path.join(golden_dir, "make_ref_se_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    g = np.load(f"{golden_dir}/ref_cuda_se.npz")
    for h, c, r in gen.SHAPES:
        x, wr, we = gen.se_case(h, c, r)
        pooled, out = so.se_module(x, wr, we)
        key = f"se_{h}_{c}_{r}"
        assert (pooled[0] - _t(g[key + "_pooled"])).abs().max() < 1e-5, key
        head = torch.stack([out[0, 0], out[0, 1], out[0, c - 1]])
        assert (head - _t(g[key + "_out_head"])).abs().max() < 2e-5, key
        s, sa = g[key + "_out_sum"]
        assert abs(sa - out.double().abs().sum().item()) / sa < 1e-5, key


def test_patch_merging_gathers_the_four_neighbours():
    """Channel block q of merged token (h, w) is input token (2h + q % 2, 2w + q // 2)
    (python/models/swin_transformer/swin_patch_merge.py:39-44); with an identity-like reduction and no affine the
    result is the LayerNorm of that concatenation."""
    cfg = so.SwinConfig(res=4, dim=2)
    x = torch.arange(4 * 4 * 2, dtype=torch.float32).reshape(16, 2)
    m = dict(norm_g=torch.ones(8), norm_b=torch.zeros(8), reduction_w=torch.eye(8)[:, :4])
    got = so.swin_patch_merge(cfg, x, m)
    assert got.shape == (4, 4)
    X = x.reshape(4, 4, 2)
    for h in range(2):
        for w in range(2):
            row = torch.cat([X[2 * h + q % 2, 2 * w + q // 2] for q in range(4)])
            ln = (row - row.mean()) / torch.sqrt(row.var(unbiased=False) + cfg.eps)
            assert torch.allclose(got[h * 2 + w], ln[:4], atol=1e-5)
