"""The C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with status codes before touching a device (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

from souffle_models_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "souffle_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(souffle_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_loads():
    path = build.build()
    assert os.path.exists(path)
    lib = _lib.load()
    assert lib.souffle_abi_version() >= 1


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    names = _declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    for n in _lib.SIGNATURES:
        assert n in names, f"{n} bound in python but not declared in the header"


def test_struct_layout_matches_header():
    assert C.sizeof(_lib.BertDesc) == 4 * 26
    assert C.sizeof(_lib.BertLayerWeights) == 8 * 12
    assert C.sizeof(_lib.LstmDesc) == 4 * 5
    assert C.sizeof(_lib.SwinDesc) == 4 * 11 and C.sizeof(_lib.SwinWeights) == 8 * 13


def test_argument_errors_need_no_device():
    lib = _lib.load()
    assert lib.souffle_bert_forward(None, None, None, None, None) == 7
    assert b"null plan" in lib.souffle_last_error()
    d = _lib.BertDesc(batch=1, seq=100, heads=12, head_dim=64, ffn=3072, n_layers=1)
    w = (_lib.BertLayerWeights * 1)()
    h = C.c_void_p()
    assert lib.souffle_bert_plan_create(C.byref(d), w, C.byref(h)) == 1       # seq not a multiple of 16
    assert b"seq" in lib.souffle_last_error()
    d.seq, d.head_dim = 128, 32
    assert lib.souffle_bert_plan_create(C.byref(d), w, C.byref(h)) == 1
    d.head_dim, d.n_layers = 64, 13
    assert lib.souffle_bert_plan_create(C.byref(d), w, C.byref(h)) == 1
    assert lib.souffle_gemm_f16(None, None, None, 16, 100, 64, None, 0, None) == 1   # N % 64
    assert lib.souffle_gemm_f16(None, None, None, 16, 128, 64, None, 0, None) == 2   # null pointers
    assert lib.souffle_swin_mlp_forward(None, None, None, None, None, 256, 500, 2048, None, 0, None) == 1
    assert lib.souffle_bert_plan_destroy(None) == 0
    ld = _lib.LstmDesc(layers=0, hidden=256, steps=100)
    assert lib.souffle_lstm_plan_create(C.byref(ld), None, None, None, C.byref(h)) in (1, 7)


def test_python_mirror_validates_before_calling():
    torch = pytest.importorskip("torch")
    from souffle_models_b200 import bert, swin
    x = torch.zeros(1, 128, 768, dtype=torch.float16)
    with pytest.raises(ValueError):
        bert.souffle_bert_layer(x, x, x, x, x, 7)           # unsupported opt level
    with pytest.raises(ValueError):
        bert.souffle_bert_layer(x, x, x, x, x, 3)           # CPU tensors
    with pytest.raises(ValueError):
        swin.swin_ffn(x[0], x[0], 1, 2, 3)


def test_persistent_kernels_do_not_spill():
    usage = build.resource_usage()
    mega = {k: v for k, v in usage.items() if "souffle_megakernel" in k}
    lstm = {k: v for k, v in usage.items() if "souffle_lstm_wavefront" in k}
    stages = {k: v for k, v in usage.items() if any(n in k for n in ("gemm_stage_ool", "ln_stage_ool", "attn_swin_stage",
                                                                     "ln_row_wide", "ln_gather_rows", "ln_stage_direct", "attn_store_probs", "attn_copy_probs"))}
    assert len(mega) == 4 and lstm and len(stages) == 8
    for k, (regs, st, ld) in {**mega, **lstm, **stages}.items():
        # A kernel may keep a few words of its per-stage dispatcher on the stack across its calls of out-of-line
        # functions: that code runs once per stage.  The stage functions themselves must stay clean.
        # (the opt-in CTA-pair build, ILi3E, is allowed twice that)
        limit = (64 if "ILi3E" in k else 32) if "souffle_megakernel" in k else 0
        assert st <= limit and ld <= limit, f"{k} spills ({st} B stores, {ld} B loads, {regs} registers)"
    assert all(v[0] <= 168 for v in mega.values())    # 384 threads per CTA leave 168 registers per thread


def test_packed_parameter_block_layout():
    """Offsets of the reference's packed 12-layer parameter block (cpp/bert/bert_base_impl.cu:536-572): host-only
    arithmetic, checked on a made-up base address."""
    import ctypes as C
    from souffle_models_b200 import _lib
    lib = _lib.load()
    w, mask, n = _lib.BertLayerWeights(), C.c_void_p(), C.c_size_t()
    base, B, S, H, F = 0x10000, 1, 384, 768, 3072
    assert lib.souffle_bert_packed_weights(base, B, S, H, F, C.byref(w), C.byref(mask), C.byref(n)) == 0
    assert n.value == 7235328 * 2                      # the reference's model size in halves (bert_base_impl.cu:279)
    assert mask.value == base
    off = lambda p: (p - base) // 2
    m = B * S * S
    assert off(w.qkv_w) == m and off(w.proj_w) == m + 3 * H * H and off(w.fc1_w) == m + 4 * H * H
    assert off(w.fc2_w) == m + 4 * H * H + H * F
    v = m + 4 * H * H + 2 * H * F                      # thirteen vectors follow the twelve H x H blocks
    assert [off(p) - v for p in (w.qkv_b, w.proj_b, w.ln1_g, w.ln1_b, w.fc1_b, w.fc2_b, w.ln2_g, w.ln2_b)] == \
        [0, 3 * H, 4 * H, 5 * H, 6 * H, 6 * H + F, 7 * H + F, 8 * H + F]
    assert lib.souffle_bert_packed_weights(base, 1, 3, H, F, None, None, None) != 0      # mask would break the alignment
