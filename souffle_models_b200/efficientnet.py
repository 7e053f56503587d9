"""EfficientNet squeeze-and-excite module: host-side mirror of the reference binding
(cpp/efficientnet/efficientnet_se_module_binding.cu:164-233) over souffle_se_module_forward."""
from typing import Dict, List

import torch

from . import _lib

_ws: Dict[int, torch.Tensor] = {}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes: int) -> torch.Tensor:
    dev = torch.cuda.current_device()
    if dev not in _ws or _ws[dev].numel() < nbytes:
        lib = _lib.load()
        if dev in _ws:          # the old block goes back to the allocator: the library must not trust its address any more
            lib.souffle_workspace_forget(_ws[dev].data_ptr())
        _ws[dev] = torch.zeros(int(nbytes), dtype=torch.uint8, device="cuda")
        lib.souffle_workspace_forget(_ws[dev].data_ptr())      # fresh memory, whatever lived at this address before
    return _ws[dev]


def se_module(x: torch.Tensor, se_reduce_weight: torch.Tensor, se_expand_weight: torch.Tensor, check: bool = True) -> List[torch.Tensor]:
    """x [B, C, H, W] fp32 CUDA, se_reduce_weight [R, C], se_expand_weight [C, R] -> [pooled [B, C], out [B, C, H, W]] with
    out = x + sigmoid(W_e . swish(W_r . mean_hw(x))) broadcast over H, W (the reference adds the gate,
    cpp/efficientnet/kernels/se_module_global_fused.cu:434-436)."""
    for name, t in (("input", x), ("se_reduce_weight", se_reduce_weight), ("se_expand_weight", se_expand_weight)):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous fp32 CUDA tensor")
    if x.dim() != 4:
        raise ValueError("input must be [batch, channels, height, width]")
    B, Cc, H, W = x.shape
    R = se_reduce_weight.shape[0]
    if tuple(se_reduce_weight.shape) != (R, Cc) or tuple(se_expand_weight.shape) != (Cc, R):
        raise ValueError("se_reduce_weight must be [R, C] and se_expand_weight [C, R]")
    lib = _lib.load()
    out = torch.empty_like(x)
    pooled = torch.empty(B, Cc, dtype=torch.float32, device=x.device)
    ws = _workspace(lib.souffle_se_module_workspace_bytes(B, Cc, H, W))
    _lib.check(lib.souffle_se_module_forward(x.data_ptr(), se_reduce_weight.data_ptr(), se_expand_weight.data_ptr(), out.data_ptr(),
                                             pooled.data_ptr(), B, Cc, H, W, R, ws.data_ptr(), ws.numel(), _stream_ptr()))
    if check:
        _lib.check(lib.souffle_workspace_status(ws.data_ptr(), _stream_ptr()))
    return [pooled, out]


def torch_dispatch_efficientnet_se_module_v2_short_cut_fused(input: torch.Tensor, se_reduce_weight: torch.Tensor,
                                                             se_expand_weight: torch.Tensor, opt_level: int = 0) -> List[torch.Tensor]:
    """Drop-in for the reference entry point of the same name (efficientnet_se_module_binding.cu:164-227): returns
    [reduce_output [B, C], se_short_cut_add].  The reference declares the second tensor as [B, H, W, C] but fills it in
    NCHW order (se_module_global_fused.cu:428-436); the same memory is returned under the same declared shape.  Every
    opt_level runs the one fused launch; any shape is accepted (the reference dispatches ten fixed ones)."""
    pooled, out = se_module(input, se_reduce_weight, se_expand_weight)
    B, Cc, H, W = input.shape
    return [pooled, out.view(B, H, W, Cc)]
