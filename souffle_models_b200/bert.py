"""Host-side mirror of the reference's BERT bindings over the C ABI.

`souffle_bert_layer` keeps the name, positional signature and six-tensor return of
cpp/bert/bert_binding.cu:23-46,534-540; `BertEncoder` is the plan-based interface the
benchmark configs use (any batch, 1..12 layers, length masks).  torch is used only for
device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, List, Optional, Sequence, Union

import torch

from . import _lib

STD, REF_COMPAT = 0, 1
_BUF = dict(qkv=0, probs=1, ctx=2, ln1=3, fc1=4)
_VEC_KEYS = ("qkv_b", "proj_b", "ln1_g", "ln1_b", "fc1_b", "fc2_b", "ln2_g", "ln2_b")
_MAT_KEYS = ("qkv_w", "proj_w", "fc1_w", "fc2_w")


def _stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check_f16_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.float16:
        raise ValueError(f"{name} must be float16")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


class BertEncoder:
    """A plan: `n_layers` encoder layers of fixed (batch, seq) fused into one launch."""

    def __init__(self, batch: int, seq: int, heads: int, head_dim: int, ffn: int,
                 layers: Sequence[Dict[str, torch.Tensor]], variant: int = STD, eps: Optional[float] = None,
                 keep_probs: bool = False, tuning: Optional[Dict[str, int]] = None):
        lib = _lib.load()
        self.batch, self.seq, self.heads, self.head_dim, self.ffn = batch, seq, heads, head_dim, ffn
        self.hidden = heads * head_dim
        self.variant = variant
        if eps is None:
            eps = 1e-12 if variant == STD else 1e-5
        d = _lib.BertDesc(batch=batch, seq=seq, heads=heads, head_dim=head_dim, ffn=ffn, n_layers=len(layers),
                          variant=variant, keep_probs=int(keep_probs), eps=eps)
        for k, v in (tuning or {}).items():
            setattr(d, k, v)
        arr = (_lib.BertLayerWeights * len(layers))()
        for i, w in enumerate(layers):
            for k in _MAT_KEYS:
                _check_f16_cuda(w[k], k)
                setattr(arr[i], k, w[k].data_ptr())
            for k in _VEC_KEYS:
                t = w.get(k)
                if t is not None:
                    _check_f16_cuda(t, k)
                setattr(arr[i], k, t.data_ptr() if t is not None else None)
        self._h = C.c_void_p()
        _lib.check(lib.souffle_bert_plan_create(C.byref(d), arr, C.byref(self._h)))
        self._lib = lib

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.souffle_bert_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, x: torch.Tensor, seq_lens: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: fp16 CUDA [B,S,H] (or [B*S,H]); seq_lens: int32 CUDA [B] or None.  Asynchronous."""
        _check_f16_cuda(x, "x")
        if x.numel() != self.batch * self.seq * self.hidden:
            raise ValueError(f"x has {x.numel()} elements, plan expects {self.batch}x{self.seq}x{self.hidden}")
        if out is None:
            out = torch.empty_like(x)
        lens_ptr = None
        if seq_lens is not None:
            if seq_lens.dtype != torch.int32 or not seq_lens.is_cuda or seq_lens.numel() != self.batch:
                raise ValueError("seq_lens must be an int32 CUDA tensor of length batch")
            lens_ptr = seq_lens.data_ptr()
        _lib.check(self._lib.souffle_bert_forward(self._h, x.data_ptr(), lens_ptr, out.data_ptr(), _stream_ptr()))
        return out

    def forward_host(self, x_host: torch.Tensor, seq_lens_host: Optional[torch.Tensor], y_host: torch.Tensor,
                     wait: bool = True) -> None:
        """Host buffers in and out (pinned preferred).  With wait=False the call returns at once and consecutive
        calls overlap their copies with one another's compute; y_host is complete once the current stream has
        caught up (x_host and y_host must be left alone until then)."""
        lens_ptr = seq_lens_host.data_ptr() if seq_lens_host is not None else None
        fn = self._lib.souffle_bert_forward_host if wait else self._lib.souffle_bert_forward_host_async
        _lib.check(fn(self._h, x_host.data_ptr(), lens_ptr, y_host.data_ptr(), _stream_ptr()))

    def status(self) -> None:
        """Synchronises and raises SouffleError if a device-side wait expired."""
        _lib.check(self._lib.souffle_bert_plan_status(self._h))

    def info(self) -> Dict[str, int]:
        a, b, c = C.c_int(), C.c_int(), C.c_int()
        _lib.check(self._lib.souffle_bert_plan_info(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return dict(launches=a.value, grid=b.value, stages=c.value, pairs=int(self._lib.souffle_bert_plan_uses_pairs(self._h)))

    def stage_info(self, index: int) -> Dict[str, int]:
        """Tiling of stage `index`: type (0 GEMM, 1 attention, 2 LayerNorm), tile rows/columns, split-K, items, ring slots."""
        out = (C.c_int * 6)()
        _lib.check(self._lib.souffle_bert_plan_stage_info(self._h, index, out))
        return dict(type=out[0], bm=out[1], bn=out[2], splitk=out[3], items=out[4], slots=out[5])

    def read_profile(self) -> torch.Tensor:
        """[stages + 1, grid, 16] int64 SM-clock stamps / role cycle totals of the last launch
        (needs tuning={'profile': 1}; layout in include/souffle_b200.h)."""
        i = self.info()
        out = torch.zeros(i["stages"] + 1, i["grid"], 16, dtype=torch.int64)    # last record: kernel entry/prologue/exit
        _lib.check(self._lib.souffle_bert_plan_read_profile(self._h, out.data_ptr(), out.numel()))
        return out

    def buffer(self, name: str) -> torch.Tensor:
        """Copy of a last-layer stage output (see SouffleBertBuffer in the header)."""
        B, S, h, d, H, F = self.batch, self.seq, self.heads, self.head_dim, self.hidden, self.ffn
        shape = dict(qkv=(3, B, h, S, d), probs=(B * h, S, S), ctx=(B * S, H), ln1=(B * S, H), fc1=(B * S, F))[name]
        out = torch.empty(shape, dtype=torch.float16, device="cuda")
        _lib.check(self._lib.souffle_bert_plan_copy_buffer(self._h, _BUF[name], out.data_ptr(), out.numel() * 2,
                                                           _stream_ptr()))
        return out


_layer_cache: Dict[tuple, tuple] = {}    # key -> (plan, weak references to the weight tensors the plan was built from)


def souffle_bert_layer(src: torch.Tensor, qkv_weight: torch.Tensor, attn_fc_weight: torch.Tensor,
                       feed_forward_fc1_weight: torch.Tensor, feed_forward_fc2_weight: torch.Tensor,
                       opt_level: int) -> List[torch.Tensor]:
    """Drop-in for bert_binding.souffle_bert_layer (cpp/bert/bert_binding.cu:23-46, 534).

    src [1,S,768] fp16, weights in [K][N] layout; returns [output_qkv, query_key_output,
    attn_value_output, attn_fc_output, feed_forward_fc1_output, feed_forward_fc2_output].
    Computes what the reference's fused kernels compute (REF_COMPAT variant).  Every
    opt_level 0..4 runs the same single fused launch; other values raise, where the reference
    prints and returns zeros (bert_binding.cu:529-531).  The plan (repacked weights) is cached
    for as long as the same weight tensors, unmodified, are passed again.
    """
    if opt_level not in (0, 1, 2, 3, 4):
        raise ValueError(f"opt level {opt_level} not supported")
    for name, t in (("src", src), ("qkv_weight", qkv_weight), ("attn_fc_weight", attn_fc_weight),
                    ("feed_forward_fc1_weight", feed_forward_fc1_weight),
                    ("feed_forward_fc2_weight", feed_forward_fc2_weight)):
        _check_f16_cuda(t, name)
    B, S, H = src.shape
    F = feed_forward_fc1_weight.shape[1]
    heads = H // 64
    weights = (qkv_weight, attn_fc_weight, feed_forward_fc1_weight, feed_forward_fc2_weight)
    key = (B, S, H, F) + tuple((t.data_ptr(), t._version) for t in weights)
    hit = _layer_cache.get(key)
    # an address and a version can come back with other contents once a tensor has been freed: the entry only counts
    # while the very tensor objects it was built from are alive
    if hit is not None and not all(r() is t for r, t in zip(hit[1], weights)):
        _layer_cache.pop(key)[0].close()
        hit = None
    if hit is None:
        if len(_layer_cache) >= 4:
            _layer_cache.pop(next(iter(_layer_cache)))[0].close()
        w = dict(qkv_w=qkv_weight, proj_w=attn_fc_weight, fc1_w=feed_forward_fc1_weight,
                 fc2_w=feed_forward_fc2_weight)
        hit = (BertEncoder(B, S, heads, 64, F, [w], variant=REF_COMPAT, keep_probs=True), tuple(weakref.ref(t) for t in weights))
        _layer_cache[key] = hit
    enc = hit[0]
    out = enc.forward(src).reshape(B * S, H)
    # the copies of the intermediates are queued behind the launch while it runs; one wait at the end
    outs = [enc.buffer("qkv").reshape(3 * B, heads, S, 64), enc.buffer("probs"), enc.buffer("ctx"),
            enc.buffer("ln1"), enc.buffer("fc1"), out]
    enc.status()                                   # blocks, as the reference call does (bert_binding.cu:532)
    return outs


_PACKED_ORDER = ("qkv_w", "proj_w", "fc1_w", "fc2_w", "qkv_b", "proj_b", "ln1_g", "ln1_b", "fc1_b", "fc2_b", "ln2_g", "ln2_b")


def packed_block_size(batch: int, seq: int, hidden: int = 768, ffn: int = 3072) -> int:
    """Number of fp16 values in the reference's packed parameter block (cpp/bert/bert_base_impl.cu:536-538)."""
    n = C.c_size_t()
    _lib.check(_lib.load().souffle_bert_packed_weights(None, batch, seq, hidden, ffn, None, None, C.byref(n)))
    return n.value // 2


def unpack_weights(blob: torch.Tensor, batch: int, seq: int, hidden: int = 768, ffn: int = 3072):
    """Views into the reference's packed parameter block (cpp/bert/bert_base_impl.cu:536-572): returns
    (mask[batch, seq, seq], layer dict with the keys BertEncoder takes).  Nothing is copied; the offsets come
    from souffle_bert_packed_weights."""
    if blob.dtype != torch.float16 or blob.dim() != 1 or not blob.is_contiguous():
        raise ValueError("the packed block must be a contiguous 1-D fp16 tensor")
    if blob.numel() < packed_block_size(batch, seq, hidden, ffn):
        raise ValueError(f"packed block holds {blob.numel()} values, {packed_block_size(batch, seq, hidden, ffn)} needed")
    w, mask_ptr = _lib.BertLayerWeights(), C.c_void_p()
    _lib.check(_lib.load().souffle_bert_packed_weights(blob.data_ptr(), batch, seq, hidden, ffn, C.byref(w), C.byref(mask_ptr), None))
    shapes = dict(qkv_w=(3, hidden, hidden), proj_w=(hidden, hidden), fc1_w=(hidden, ffn), fc2_w=(ffn, hidden), qkv_b=(3, hidden),
                  proj_b=(hidden,), ln1_g=(hidden,), ln1_b=(hidden,), fc1_b=(ffn,), fc2_b=(hidden,), ln2_g=(hidden,), ln2_b=(hidden,))
    base = blob.data_ptr()

    def view(ptr, shape):
        off = (ptr - base) // 2
        n = 1
        for d in shape:
            n *= d
        return blob[off:off + n].view(*shape)

    layer = {k: view(getattr(w, k), shapes[k]) for k in _PACKED_ORDER}
    return view(mask_ptr.value, (batch, seq, seq)), layer


def souffle_bert_base(model: Optional[torch.Tensor] = None, src: Optional[torch.Tensor] = None) -> Union[int, torch.Tensor]:
    """Drop-in for souffle_bert_base.souffle_bert_base() (cpp/bert/bert_base_impl.cu:277-308): a 12-layer
    BERT-base encoder at batch 1, sequence 384, all layers on one parameter set, run as one launch.
    Without arguments the parameters and the input are zero-filled as in the reference (which has its file
    reads commented out, :279-283) and 0 is returned like there.  With `model` (the packed block of
    :536-572 as an fp16 CUDA tensor, see unpack_weights) and `src` [384, 768] the encoder output is returned;
    sequence lengths are taken from the first row of the block's mask."""
    B, S, H, F = 1, 384, 768, 3072
    if model is None:
        z = lambda *s: torch.zeros(*s, dtype=torch.float16, device="cuda")
        layer = dict(qkv_w=z(3, H, H), qkv_b=z(3, H), proj_w=z(H, H), proj_b=z(H), ln1_g=z(H) + 1, ln1_b=z(H),
                     fc1_w=z(H, F), fc1_b=z(F), fc2_w=z(F, H), fc2_b=z(H), ln2_g=z(H) + 1, ln2_b=z(H))
        lens, x = None, z(1, S, H)
    else:
        mask, layer = unpack_weights(model, B, S, H, F)
        lens = (mask[:, 0, :] > 0).sum(dim=-1).to(torch.int32)
        x = (src if src is not None else torch.zeros(S, H, dtype=torch.float16, device="cuda")).reshape(1, S, H)
    enc = BertEncoder(B, S, 12, 64, F, [layer] * 12, variant=STD, eps=1e-6)
    y = enc.forward(x, lens)
    enc.status()
    enc.close()
    return 0 if model is None else y.reshape(S, H)
