"""Host-side mirror of the reference's Swin bindings over the C ABI
(cpp/swin_transformer/swin_transformer_binding.cu:62-289, swin_trans_fc2_binding.cu:19-61)."""
from __future__ import annotations

import ctypes as C
from typing import List

import torch

from . import _lib
from .bert import _check_f16_cuda, _stream_ptr

_ws = {}


def _workspace(nbytes: int = 0) -> torch.Tensor:
    """Per-device scratch for the plan-less entry points (barrier words, then split-K planes); grows on demand."""
    dev = torch.cuda.current_device()
    need = max(int(nbytes), int(_lib.load().souffle_gemm_workspace_bytes()))
    if dev not in _ws or _ws[dev].numel() < need:
        if dev in _ws:          # the old block goes back to the allocator: the library must not trust its address any more
            _lib.load().souffle_workspace_forget(_ws[dev].data_ptr())
        _ws[dev] = torch.zeros(need, dtype=torch.uint8, device="cuda")
        _lib.load().souffle_workspace_forget(_ws[dev].data_ptr())      # fresh memory, whatever lived at this address before
    return _ws[dev]


def gemm(a: torch.Tensor, w_kn: torch.Tensor, check: bool = True) -> torch.Tensor:
    """c[M,N] = a[M,K] . w[K,N], fp16 in/out, fp32 accumulate."""
    _check_f16_cuda(a, "a")
    _check_f16_cuda(w_kn, "w")
    M, K = a.shape
    K2, N = w_kn.shape
    if K2 != K:
        raise ValueError(f"inner dimensions differ: {K} vs {K2}")
    c = torch.empty(M, N, dtype=torch.float16, device=a.device)
    ws = _workspace()
    lib = _lib.load()
    _lib.check(lib.souffle_gemm_f16(a.data_ptr(), w_kn.data_ptr(), c.data_ptr(), M, N, K, ws.data_ptr(),
                                    ws.numel(), _stream_ptr()))
    if check:
        _lib.check(lib.souffle_workspace_status(ws.data_ptr(), _stream_ptr()))
    return c


def swin_ffn(src: torch.Tensor, weight: torch.Tensor, M: int, N: int, K: int) -> torch.Tensor:
    """swin_transformer_binding.swin_ffn (swin_transformer_binding.cu:62-100): one GEMM.  The
    reference only accepts (M,N,K) in {(256,2048,512), (256,512,2048)}; any K, N multiple of 64 works here."""
    if tuple(src.shape) != (M, K) or tuple(weight.shape) != (K, N):
        raise ValueError("src must be [M,K] and weight [K,N]")
    return gemm(src, weight)


def swin_trans_fc2(src: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """swin_trans_fc2.swin_trans_fc2 (swin_trans_fc2_binding.cu:19-55): src [1,256,2048] x weight [2048,512]."""
    s2 = src.reshape(-1, src.shape[-1])
    return gemm(s2, weight).reshape(*src.shape[:-1], weight.shape[1])


def swin_fused_feed_mlp(src: torch.Tensor, fc1_weight: torch.Tensor, fc2_weight: torch.Tensor,
                        check: bool = True) -> List[torch.Tensor]:
    """swin_transformer_binding.swin_fused_feed_mlp (swin_transformer_binding.cu:155-209):
    returns [fc1_output[M,F], fc2_output[M,C]] from one launch with a grid barrier between the GEMMs."""
    for n, t in (("src", src), ("fc1_weight", fc1_weight), ("fc2_weight", fc2_weight)):
        _check_f16_cuda(t, n)
    M, Cc = src.shape
    F = fc1_weight.shape[1]
    if tuple(fc1_weight.shape) != (Cc, F) or tuple(fc2_weight.shape) != (F, Cc):
        raise ValueError("fc1_weight must be [C,F] and fc2_weight [F,C]")
    hidden = torch.empty(M, F, dtype=torch.float16, device=src.device)
    out = torch.empty(M, Cc, dtype=torch.float16, device=src.device)
    lib = _lib.load()
    ws = _workspace(lib.souffle_swin_mlp_workspace_bytes(M, Cc, F))
    _lib.check(lib.souffle_swin_mlp_forward(src.data_ptr(), fc1_weight.data_ptr(), fc2_weight.data_ptr(),
                                            hidden.data_ptr(), out.data_ptr(), M, Cc, F, ws.data_ptr(), ws.numel(),
                                            _stream_ptr()))
    if check:
        _lib.check(lib.souffle_workspace_status(ws.data_ptr(), _stream_ptr()))
    return [hidden, out]


def _bench(fn, num_warmup: int, num_bench: int, repeat: int) -> float:
    """Minimum over `num_bench` rounds of the mean latency in microseconds of `repeat` calls, timed with
    CUDA events after `num_warmup` calls (cpp/souffle_utils/cuda_utils.h:102-136)."""
    for _ in range(num_warmup):
        fn()
    best = float("inf")
    for _ in range(max(1, num_bench)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(max(1, repeat)):
            fn()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1000.0 / max(1, repeat))
    return best


def bench_swin_ffn(M: int, N: int, K: int, num_warmup: int, num_bench: int, repeat: int) -> float:
    """swin_transformer_binding.bench_swin_ffn (swin_transformer_binding.cu:102-152): latency in microseconds of
    one [M,K] x [K,N] product on random operands."""
    src = torch.rand(M, K, device="cuda").half()
    w = torch.rand(K, N, device="cuda").half()
    return _bench(lambda: gemm(src, w, check=False), num_warmup, num_bench, repeat)


def bench_swin_fused_feed_mlp(src: torch.Tensor, fc1_weight: torch.Tensor, fc2_weight: torch.Tensor, num_warmup: int,
                              repeat: int, num_bench: int) -> float:
    """swin_transformer_binding.bench_swin_fused_feed_mlp (swin_transformer_binding.cu:211-273): the same
    positional arguments -- the three tensors of swin_fused_feed_mlp, then num_warmup, repeat, num_bench in the
    order the binding declares them (:214-217) and hands them to the timing loop (:271) -- and the same result,
    microseconds per fused fc1 -> fc2 launch.  The reference asserts the shape [256,512] x [512,2048] x [2048,512];
    any M and multiples of 64 for the two widths work here."""
    return _bench(lambda: swin_fused_feed_mlp(src, fc1_weight, fc2_weight, check=False), num_warmup, repeat, num_bench)


def layernorm(partial: torch.Tensor, resid=None, bias=None, gamma=None, beta=None, eps: float = 1e-5,
              check: bool = True) -> torch.Tensor:
    """out = LayerNorm(sum over planes of partial[P,M,N] (fp32) + bias + resid) * gamma + beta -> fp16 [M,N]."""
    if partial.dtype != torch.float32 or not partial.is_cuda or partial.dim() != 3:
        raise ValueError("partial must be a float32 CUDA tensor [P, M, N]")
    P, M, N = partial.shape
    out = torch.empty(M, N, dtype=torch.float16, device=partial.device)
    ws = _workspace()
    lib = _lib.load()
    ptr = lambda t: t.data_ptr() if t is not None else None
    _lib.check(lib.souffle_layernorm_forward(partial.data_ptr(), P, ptr(bias), ptr(resid), ptr(gamma), ptr(beta),
                                             out.data_ptr(), M, N, eps, ws.data_ptr(), ws.numel(), _stream_ptr()))
    if check:
        _lib.check(lib.souffle_workspace_status(ws.data_ptr(), _stream_ptr()))
    return out


class SwinBlock:
    """Plan for one Swin block, or for a chain of blocks run as one launch (see SouffleSwinDesc in the header).
    `params` is a weights dict with the keys of oracle.souffle_oracle.make_swin_params (fp16 CUDA tensors, matrices
    [K][N]) or a list of such dicts, one per block; even-numbered blocks use `shift`, odd-numbered ones `shift_alt`.
    `merge` (dict with norm_g, norm_b [4*dim] and reduction_w [4*dim, 2*dim]) appends the patch merging that ends a
    stage of the network (python/models/swin_transformer/swin_patch_merge.py:1-17) to the same launch; the output is
    then [batch*(res/2)^2, 2*dim]."""

    KEYS = ("ln1_g", "ln1_b", "qkv_w", "qkv_b", "rel_bias", "proj_w", "proj_b", "ln2_g", "ln2_b", "fc1_w", "fc1_b",
            "fc2_w", "fc2_b")

    def __init__(self, batch: int, res: int, dim: int, heads: int, window: int, shift: int, params, mlp_ratio: int = 4,
                 eps: float = 1e-5, shift_alt: int = 0, merge=None):
        lib = _lib.load()
        self.batch, self.res, self.dim = batch, res, dim
        self.out_shape = (batch * res * res, dim) if merge is None else (batch * (res // 2) ** 2, 2 * dim)
        blocks = list(params) if isinstance(params, (list, tuple)) else [params]
        d = _lib.SwinDesc(batch=batch, res=res, dim=dim, heads=heads, window=window, shift=shift, mlp_ratio=mlp_ratio, eps=eps,
                          n_blocks=len(blocks), shift_alt=shift_alt)
        ws = (_lib.SwinWeights * len(blocks))()
        self._keep = blocks
        for w, blk in zip(ws, blocks):
            for k in self.KEYS:
                t = blk.get(k)
                if t is not None:
                    _check_f16_cuda(t, k)
                setattr(w, k, t.data_ptr() if t is not None else None)
        mg = None
        if merge is not None:
            mg = _lib.SwinMerge()
            for k in ("norm_g", "norm_b", "reduction_w"):
                t = merge.get(k)
                if t is not None:
                    _check_f16_cuda(t, k)
                setattr(mg, k, t.data_ptr() if t is not None else None)
            self._keep = (blocks, merge)
        self._h = C.c_void_p()
        _lib.check(lib.souffle_swin_stage_plan_create(C.byref(d), ws, C.byref(mg) if mg is not None else None,
                                                      C.byref(self._h)))
        self._lib = lib

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.souffle_swin_block_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: fp16 CUDA [batch*res*res, dim]; asynchronous."""
        _check_f16_cuda(x, "x")
        if x.numel() != self.batch * self.res * self.res * self.dim:
            raise ValueError("x has the wrong number of elements for this plan")
        y = torch.empty(self.out_shape, dtype=torch.float16, device=x.device)
        _lib.check(self._lib.souffle_swin_block_forward(self._h, x.data_ptr(), y.data_ptr(), _stream_ptr()))
        return y

    def status(self) -> None:
        _lib.check(self._lib.souffle_swin_block_plan_status(self._h))


def swin_stage(x: torch.Tensor, blocks, merge=None, batch: int = 1, res: int = 14, heads: int = 16, window: int = 7,
               shift: int = 3, mlp_ratio: int = 4, eps: float = 1e-5) -> torch.Tensor:
    """A stage of the network as one launch: `blocks` (list of weight dicts) with shifts 0, `shift`, 0, ... and, with
    `merge`, the patch merging after them.  The reference runs this part of the model as separate TVM kernels, 226 for
    the whole model (python/models/tee:1)."""
    plan = SwinBlock(batch, res, x.shape[-1], heads, window, 0, list(blocks), mlp_ratio=mlp_ratio, eps=eps, shift_alt=shift,
                     merge=merge)
    try:
        y = plan.forward(x.reshape(-1, x.shape[-1]))
        plan.status()
    finally:
        plan.close()
    return y
