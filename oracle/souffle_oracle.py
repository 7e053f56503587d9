"""CPU restatement (fp32, torch-CPU / numpy) of the reference's fused encoder paths.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; only the
parity tests, the smoke check and the bench's `cpu_baseline` / `--impl reference` legs do,
and there only as the checker or as the timed CPU arm, never as the product path.

Parity pin status
-----------------
* BERT layer structure (fused QKV -> per-head bmm -> softmax -> bmm -> merge heads ->
  fc + residual -> LayerNorm -> FFN -> residual -> LayerNorm) is pinned against the
  reference's own torch modules (python/models/bert/bert_torch.py:17-56, 88-143) run on CPU;
  the vectors and the generating script live in tests/golden/.
* The reference stores no golden vectors for the fused CUDA kernels, the LSTM or Swin
  (its tests only carry tolerances), so those restatements are pinned by outputs of the
  reference CUDA kernels themselves (built from the reference sources by oracle/Makefile
  into oracle/_ref/ and run on a GPU); where such a fixture is absent the function's
  docstring says "parity unpinned".

Every function cites the reference file:line it follows (paths relative to the reference
project root).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

F32 = torch.float32


# --------------------------------------------------------------------------------------
# Configuration records (plain data; mirrored by the C structs in include/souffle_b200.h)
# --------------------------------------------------------------------------------------
@dataclass
class BertConfig:
    """Shape/variant record of one encoder layer.

    `BERT_STD` (variant="std") is the model the benchmark configs describe: scale 1/sqrt(d),
    additive length mask (1-m)*-1e4 as cpp/bert/kernels/softmax.cu:22-24, tanh-GELU as
    cpp/bert/bert_base_impl.cu:722-734, bias vectors, vector gamma/beta, eps 1e-12.
    `REF_COMPAT` (variant="ref") is what the reference's fused kernel computes
    (cpp/bert/kernels/fused_sqq_bert.cu:2934 scale 1/sqrt(hidden), ReLU
    cpp/bert/kernels/fused_sqq_feedforward.cu:2120-2133, no proj/FFN bias, LN without
    affine and eps 1e-5, cpp/bert/bert_binding.cu:115).
    """
    batch: int = 1
    seq: int = 128
    heads: int = 12
    head_dim: int = 64
    ffn: int = 3072
    variant: str = "std"

    @property
    def hidden(self) -> int:
        return self.heads * self.head_dim

    @property
    def scale(self) -> float:
        if self.variant == "ref":
            return 1.0 / math.sqrt(self.hidden)
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def eps(self) -> float:
        return 1e-5 if self.variant == "ref" else 1e-12

    @property
    def act(self) -> str:
        return "relu" if self.variant == "ref" else "gelu_tanh"


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """tanh-form GELU, cpp/bert/bert_base_impl.cu:722-734."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def _r16(t: torch.Tensor, on: bool) -> torch.Tensor:
    """Round through fp16 storage when emulating the kernel's fp16 intermediates."""
    return t.half().float() if on else t


def make_bert_weights(cfg: BertConfig, seed: int, n_layers: int = 1,
                      zero_bias: bool = True) -> List[Dict[str, torch.Tensor]]:
    """Seeded synthetic weights: N(0, 0.02) fp16 in the reference's [K][N] layout
    (cpp/bert/test_souffle_bert_layer.py:139-143), biases 0, gamma 1, beta 0.
    `zero_bias=False` draws small non-zero vectors so the bias/affine paths are exercised."""
    g = torch.Generator().manual_seed(seed)
    H, Fd = cfg.hidden, cfg.ffn
    layers = []
    for _ in range(n_layers):
        def w(*shape):
            return (torch.randn(*shape, generator=g) * 0.02).half()

        def v(n, base=0.0):
            if zero_bias:
                return torch.full((n,), base).half()
            return (base + torch.randn(n, generator=g) * 0.05).half()
        layers.append(dict(
            qkv_w=w(3, H, H), qkv_b=v(3 * H).view(3, H), proj_w=w(H, H), proj_b=v(H),
            ln1_g=v(H, 1.0), ln1_b=v(H), fc1_w=w(H, Fd), fc1_b=v(Fd),
            fc2_w=w(Fd, H), fc2_b=v(H), ln2_g=v(H, 1.0), ln2_b=v(H)))
    return layers


def make_bert_input(cfg: BertConfig, seed: int, ragged: bool = False):
    """N(0,1) fp16 activations [B,S,H]; `ragged` draws token lengths uniform in [S/4, S]."""
    g = torch.Generator().manual_seed(seed + 7919)
    x = torch.randn(cfg.batch, cfg.seq, cfg.hidden, generator=g).half()
    lens = None
    if ragged:
        lens = torch.randint(cfg.seq // 4, cfg.seq + 1, (cfg.batch,), generator=g).to(torch.int32)
    return x, lens


def layer_norm(z: torch.Tensor, gamma, beta, eps: float) -> torch.Tensor:
    """Row LayerNorm in fp32 (two-pass), cpp/bert/bert_base_impl.cu:743-781."""
    mu = z.mean(-1, keepdim=True)
    var = ((z - mu) ** 2).mean(-1, keepdim=True)
    y = (z - mu) * torch.rsqrt(var + eps)
    if gamma is not None:
        y = y * gamma.float() + beta.float()
    return y


def bert_layer(cfg: BertConfig, x: torch.Tensor, w: Dict[str, torch.Tensor],
               lens: Optional[torch.Tensor] = None, emulate_fp16: bool = False,
               scale: Optional[float] = None, act: Optional[str] = None,
               eps: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """One encoder layer in fp32 from fp16-valued inputs.

    Follows python/models/bert/bert_torch.py:36-56 (attention half) and :97-104 (FFN half);
    the returned dict carries the six stage outputs of the reference binding
    (cpp/bert/bert_binding.cu:534): qkv [3,B,h,S,d], probs [B,h,S,S], ctx [B*S,H],
    ln1 [B*S,H], fc1 [B*S,F], out [B*S,H].  `emulate_fp16` rounds each tensor that the
    CUDA path stores in fp16 so the comparison isolates arithmetic from storage rounding.
    """
    B, S, h, d, H = cfg.batch, cfg.seq, cfg.heads, cfg.head_dim, cfg.hidden
    scale = cfg.scale if scale is None else scale
    act = cfg.act if act is None else act
    eps = cfg.eps if eps is None else eps
    std = cfg.variant == "std"
    e = emulate_fp16
    X = x.float().reshape(B * S, H)
    qkv = torch.stack([X @ w["qkv_w"][j].float() + w["qkv_b"][j].float() for j in range(3)])
    qkv = _r16(qkv, e).reshape(3, B, S, h, d).permute(0, 1, 3, 2, 4)       # [3,B,h,S,d]
    q, k, v = qkv[0], qkv[1], qkv[2]
    s = (q @ k.transpose(-1, -2)) * scale                                   # [B,h,S,S]
    if lens is not None:
        m = (torch.arange(S)[None, :] < lens.to(torch.int64)[:, None]).float()   # [B,S]
        s = s + ((1.0 - m) * -10000.0)[:, None, None, :]
    p = torch.softmax(s, dim=-1)
    if e:
        # the CUDA path multiplies the UNNORMALISED probabilities, rounded to fp16, with V and divides by their fp32 sum
        pu = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        ctx = (_r16(pu, True) @ v) / pu.sum(dim=-1, keepdim=True)
    else:
        ctx = p @ v
    ctx = _r16(ctx.permute(0, 2, 1, 3).reshape(B * S, H), e)
    z1 = ctx @ w["proj_w"].float() + X          # pre-LayerNorm sums stay fp32 in the CUDA path (fp32 split-K planes)
    if std:
        z1 = z1 + w["proj_b"].float()
    ln1 = _r16(layer_norm(z1, w["ln1_g"] if std else None, w["ln1_b"] if std else None, eps), e)
    a = ln1 @ w["fc1_w"].float()
    if std:
        a = a + w["fc1_b"].float()
    a = torch.relu(a) if act == "relu" else gelu_tanh(a)
    a = _r16(a, e)
    z2 = a @ w["fc2_w"].float() + ln1
    if std:
        z2 = z2 + w["fc2_b"].float()
    out = layer_norm(z2, w["ln2_g"] if std else None, w["ln2_b"] if std else None, eps)
    return dict(qkv=qkv.contiguous(), probs=p, ctx=ctx, ln1=ln1, fc1=a, out=out)


def bert_stack(cfg: BertConfig, x: torch.Tensor, layers: Sequence[Dict[str, torch.Tensor]],
               lens: Optional[torch.Tensor] = None, emulate_fp16: bool = False) -> torch.Tensor:
    """N-layer encoder chain; the loop of cpp/bert/bert_base_impl.cu:590-678 with a
    distinct weight set per layer.  Activations pass between layers as fp16 values,
    which is what both the reference and the CUDA path store."""
    cur = x.float().reshape(cfg.batch * cfg.seq, cfg.hidden)
    for w in layers:
        cur = bert_layer(cfg, cur, w, lens, emulate_fp16)["out"]
        if emulate_fp16:
            cur = cur.half().float()
    return cur


# --------------------------------------------------------------------------------------
# LSTM wavefront
# --------------------------------------------------------------------------------------
def make_lstm_params(layers=10, hidden=256, steps=100, seed=1237):
    """fp16-valued U(-1/16, 1/16) weights in the reference's [4*layer + gate][out][in]
    layout (cpp/lstm/lstm_reuse_shared_memory.cu:200-208 indexes weight[row, :] . x)."""
    g = torch.Generator().manual_seed(seed)
    w_in = ((torch.rand(4 * layers, hidden, hidden, generator=g) - 0.5) / 8.0).half()
    w_st = ((torch.rand(4 * layers, hidden, hidden, generator=g) - 0.5) / 8.0).half()
    x = torch.randn(1, steps, hidden, generator=g).half()
    return x, w_in, w_st


def lstm_forward(x: torch.Tensor, w_in: torch.Tensor, w_st: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, ref_input_delay: bool = False) -> torch.Tensor:
    """Stacked LSTM, batch 1.  Gate order i, j, f, o; c' = c*sigmoid(f+1) + sigmoid(i)*tanh(j);
    h' = tanh(c')*sigmoid(o)  (python/models/lstm/tf_lstm.py:59-70;
    cpp/lstm/lstm_reuse_shared_memory.cu:309-318).  Weights are [out][in].

    `ref_input_delay=True` reproduces the reference kernel's feeding order, where layer 0 at
    wavefront step s consumes x[s-1] (zeros at s=0) and x[T-1] is never consumed
    (cpp/lstm/lstm_reuse_shared_memory.cu:324-326).  Returns the top layer's h per step [1,T,H].
    Pinned in that form against the output of the reference kernel on a GPU
    (tests/golden/ref_cuda_lstm_swin.npz: agreement to 2e-7).
    """
    T, Hd = x.shape[1], x.shape[2]
    L = w_in.shape[0] // 4
    Wi = w_in.float().reshape(L, 4, Hd, Hd)
    Ws = w_st.float().reshape(L, 4, Hd, Hd)
    b = torch.zeros(L, Hd) if bias is None else bias.float().reshape(L, Hd)
    xs = x.float()[0]
    if ref_input_delay:
        xs = torch.cat([torch.zeros(1, Hd), xs[:-1]], 0)
    c = torch.zeros(L, Hd)
    hh = torch.zeros(L, Hd)
    out = torch.zeros(T, Hd)
    for t in range(T):
        inp = xs[t]
        for l in range(L):
            g = Wi[l] @ inp + Ws[l] @ hh[l] + b[l]          # [4,Hd]
            c[l] = c[l] * torch.sigmoid(g[2] + 1.0) + torch.sigmoid(g[0]) * torch.tanh(g[1])
            hh[l] = torch.tanh(c[l]) * torch.sigmoid(g[3])
            inp = hh[l]
        out[t] = hh[L - 1]
    return out[None]


# --------------------------------------------------------------------------------------
# Swin: plain GEMMs of the C++ path and the full shifted-window block of the config
# --------------------------------------------------------------------------------------
def gemm_kn(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """C[M,N] = A[M,K] . W[K,N]: cpp/swin_transformer/swin_transformer_binding.cu:62-100
    (`swin_ffn`) and swin_trans_fc2_binding.cu:19-55 (`swin_trans_fc2`)."""
    return a.float() @ w.float()


def swin_mlp(src: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, emulate_fp16=False):
    """fc1 -> fc2 with no bias, activation, norm or residual, exactly as
    cpp/swin_transformer/kernels/swin_fused_ffn_m256n2048k512_m256n512k2048.cu:9-769.  Pinned against that
    kernel's output on a GPU (tests/golden/ref_cuda_lstm_swin.npz; the kernel accumulates in fp16: within 1e-2)."""
    h1 = _r16(gemm_kn(src, w1), emulate_fp16)
    return h1, gemm_kn(h1, w2)


@dataclass
class SwinConfig:
    """Swin-B stage-3 block of the benchmark config: 14x14 tokens, C=512, 16 heads x 32,
    window 7, MLP ratio 4, pre-LN, tanh-GELU (python/models/swin_transformer/swin_mlp.py:91-96)."""
    res: int = 14
    dim: int = 512
    heads: int = 16
    window: int = 7
    mlp_ratio: int = 4
    eps: float = 1e-5

    @property
    def head_dim(self):
        return self.dim // self.heads


def make_swin_params(cfg: SwinConfig, seed: int, zero_bias=True):
    g = torch.Generator().manual_seed(seed)
    C, Fd = cfg.dim, cfg.dim * cfg.mlp_ratio

    def w(*s):
        return (torch.randn(*s, generator=g) * 0.02).half()

    def v(n, base=0.0):
        if zero_bias:
            return torch.full((n,), base).half()
        return (base + torch.randn(n, generator=g) * 0.05).half()
    tbl = (2 * cfg.window - 1)
    return dict(ln1_g=v(C, 1.0), ln1_b=v(C), qkv_w=w(C, 3 * C), qkv_b=v(3 * C),
                rel_bias=w(tbl * tbl, cfg.heads), proj_w=w(C, C), proj_b=v(C),
                ln2_g=v(C, 1.0), ln2_b=v(C), fc1_w=w(C, Fd), fc1_b=v(Fd), fc2_w=w(Fd, C), fc2_b=v(C))


def swin_rel_index(ws: int) -> torch.Tensor:
    """[ws*ws, ws*ws] index into the (2ws-1)^2 relative-position table: entry (p,q) is
    (dy + ws-1)*(2ws-1) + (dx + ws-1) with (dy,dx) the offset of token p from token q."""
    c = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)
    rel = c[:, :, None] - c[:, None, :]
    return (rel[0] + ws - 1) * (2 * ws - 1) + (rel[1] + ws - 1)


def swin_shift_mask(res: int, ws: int, shift: int) -> torch.Tensor:
    """[nW, ws*ws, ws*ws] additive mask (0 / -100) separating the three wrapped bands per
    axis after the cyclic shift, so tokens that were not neighbours do not attend."""
    nW = (res // ws) ** 2
    if shift == 0:
        return torch.zeros(nW, ws * ws, ws * ws)
    img = torch.zeros(res, res)
    cnt = 0
    for hs in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
        for wsl in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
            img[hs, wsl] = cnt
            cnt += 1
    win = img.reshape(res // ws, ws, res // ws, ws).permute(0, 2, 1, 3).reshape(nW, ws * ws)
    diff = win[:, None, :] - win[:, :, None]
    return torch.where(diff != 0, torch.tensor(-100.0), torch.tensor(0.0))


def swin_block(cfg: SwinConfig, x: torch.Tensor, p: Dict[str, torch.Tensor], shift: int,
               emulate_fp16: bool = False) -> torch.Tensor:
    """One pre-LN shifted-window block on [res*res, C]; structure of the Part-1..Part-8
    description in python/models/swin_transformer/swin_transformer_main.py:11-61, with the
    relative-position bias table and shift mask the benchmark config adds (absent from the
    reference's TE definitions).  parity unpinned: the reference has no runnable
    implementation of the attention half in this environment.
    `emulate_fp16` rounds every tensor the CUDA path stores in fp16 (both LayerNorm outputs, Q/K/V, the
    unnormalised probabilities, the attention output, the residual stream after the attention half, the MLP
    hidden layer), so that a comparison isolates arithmetic from storage rounding."""
    R, C, h, d, ws = cfg.res, cfg.dim, cfg.heads, cfg.head_dim, cfg.window
    e = emulate_fp16
    nwr = R // ws
    X = x.float().reshape(R * R, C)
    y = _r16(layer_norm(X, p["ln1_g"], p["ln1_b"], cfg.eps), e).reshape(R, R, C)
    if shift:
        y = torch.roll(y, shifts=(-shift, -shift), dims=(0, 1))
    win = y.reshape(nwr, ws, nwr, ws, C).permute(0, 2, 1, 3, 4).reshape(nwr * nwr, ws * ws, C)
    qkv = _r16(win @ p["qkv_w"].float() + p["qkv_b"].float(), e)
    qkv = qkv.reshape(nwr * nwr, ws * ws, 3, h, d).permute(2, 0, 3, 1, 4)       # [3,nW,h,N,d]
    q, k, v = qkv[0], qkv[1], qkv[2]
    att = (q @ k.transpose(-1, -2)) * (d ** -0.5)                                # [nW,h,N,N]
    bias = p["rel_bias"].float()[swin_rel_index(ws).reshape(-1)].reshape(ws * ws, ws * ws, h)
    att = att + bias.permute(2, 0, 1)[None] + swin_shift_mask(R, ws, shift)[:, None]
    if e:
        pu = torch.exp(att - att.max(dim=-1, keepdim=True).values)
        o = (_r16(pu, True) @ v) / pu.sum(dim=-1, keepdim=True)
    else:
        o = torch.softmax(att, -1) @ v
    o = _r16(o.permute(0, 2, 1, 3).reshape(nwr * nwr, ws * ws, C), e)
    o = o @ p["proj_w"].float() + p["proj_b"].float()
    o = o.reshape(nwr, nwr, ws, ws, C).permute(0, 2, 1, 3, 4).reshape(R, R, C)
    if shift:
        o = torch.roll(o, shifts=(shift, shift), dims=(0, 1))
    X = _r16(X + o.reshape(R * R, C), e)
    y2 = _r16(layer_norm(X, p["ln2_g"], p["ln2_b"], cfg.eps), e)
    a = _r16(gelu_tanh(y2 @ p["fc1_w"].float() + p["fc1_b"].float()), e)
    return X + a @ p["fc2_w"].float() + p["fc2_b"].float()


def make_swin_merge_params(cfg: SwinConfig, seed: int, zero_bias=True):
    g = torch.Generator().manual_seed(seed)
    C4 = 4 * cfg.dim
    if zero_bias:
        ng, nb = torch.ones(C4).half(), torch.zeros(C4).half()
    else:
        ng, nb = (1.0 + torch.randn(C4, generator=g) * 0.05).half(), (torch.randn(C4, generator=g) * 0.05).half()
    return dict(norm_g=ng, norm_b=nb, reduction_w=(torch.randn(C4, 2 * cfg.dim, generator=g) * 0.02).half())


def swin_patch_merge(cfg: SwinConfig, x: torch.Tensor, m: Dict[str, torch.Tensor]) -> torch.Tensor:
    """Patch merging on [res*res, C] -> [(res/2)^2, 2C]: channel block q of merged token (h, w) is input token
    (2h + q % 2, 2w + q // 2) (python/models/swin_transformer/swin_patch_merge.py:4-9 and the index expression at
    :39-44), LayerNorm over the 4C channels (:11, :103-118), reduction 4C -> 2C without bias (:12, :121-123)."""
    R, C = cfg.res, cfg.dim
    X = x.float().reshape(R, R, C)
    merged = torch.cat([X[0::2, 0::2], X[1::2, 0::2], X[0::2, 1::2], X[1::2, 1::2]], -1).reshape(-1, 4 * C)
    y = layer_norm(merged, m["norm_g"], m["norm_b"], cfg.eps)
    return y @ m["reduction_w"].float()


def se_module(x: torch.Tensor, w_reduce: torch.Tensor, w_expand: torch.Tensor):
    """EfficientNet squeeze-and-excite as the reference's fused kernel computes it
    (cpp/efficientnet/kernels/se_module_global_fused.cu:316-444): channel means (:360-372), reduce GEMV with
    s * sigmoid(s) (:375-398), expand GEMV with sigmoid (:401-425), and the gate ADDED to the input (:428-436).
    x [B, C, H, W], w_reduce [R, C], w_expand [C, R], fp32.  Returns (pooled [B, C], out [B, C, H, W]).
    Pinned against that kernel's own output on a GPU for the four dispatch shapes that run one channel per block
    (tests/golden/ref_cuda_se.npz, generator tests/golden/make_ref_se_golden.py; fp32 throughout: within 2e-5).
    With several channels per block the kernel's last stage reads its shared-memory copy at stride H*W although
    it was written at the padded stride (:431-436 against :344-352); for those shapes this restatement, not the
    kernel, is the module."""
    x = x.double()
    pooled = x.mean(dim=(2, 3))
    s = pooled @ w_reduce.double().t()
    r = s * torch.sigmoid(s)
    gate = torch.sigmoid(r @ w_expand.double().t())
    return pooled.float(), (x + gate[:, :, None, None]).float()
