"""Squeeze-and-excite module: the CUDA launch against the oracle on the reference's ten shapes
(cpp/efficientnet/test_efficientnet_se_module.py:13-23) and on shapes it does not dispatch."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import souffle_oracle as so  # noqa: E402

pytestmark = pytest.mark.gpu

REF_SHAPES = [(1, 112, 112, 32, 8), (1, 56, 56, 96, 4), (1, 56, 56, 144, 6), (1, 28, 28, 144, 6), (1, 28, 28, 240, 10),
              (1, 14, 14, 240, 10), (1, 14, 14, 480, 20), (1, 14, 14, 672, 28), (1, 7, 7, 672, 28), (1, 7, 7, 1152, 48)]


def _case(b, h, w, c, r, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, c, h, w, generator=g)
    wr = torch.randn(r, c, generator=g) * 0.2
    we = torch.randn(c, r, generator=g) * 0.5
    return x, wr, we


@pytest.mark.parametrize("shape", REF_SHAPES + [(2, 10, 13, 40, 5), (3, 1, 1, 8, 2), (1, 224, 224, 3, 1)])
def test_se_module_matches_oracle(shape):
    from souffle_models_b200 import efficientnet
    b, h, w, c, r = shape
    x, wr, we = _case(b, h, w, c, r, 7 + c)
    pooled, out = efficientnet.se_module(x.cuda(), wr.cuda(), we.cuda())
    want_pooled, want = so.se_module(x, wr, we)
    assert (pooled.cpu() - want_pooled).abs().max() < 1e-5
    assert (out.cpu() - want).abs().max() < 2e-5
    pooled2, out2 = efficientnet.se_module(x.cuda(), wr.cuda(), we.cuda())       # the workspace cleans itself up
    assert torch.equal(out, out2) and torch.equal(pooled, pooled2)


def test_drop_in_entry_returns_the_reference_shapes():
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "shims"))
    import efficientnet_se_module_binding as ref_name
    x, wr, we = _case(1, 14, 14, 240, 10, 3)
    pooled, out = ref_name.torch_dispatch_efficientnet_se_module_v2_short_cut_fused(x.cuda(), wr.cuda(), we.cuda(), 2)
    assert tuple(pooled.shape) == (1, 240) and tuple(out.shape) == (1, 14, 14, 240)
    _, want = so.se_module(x, wr, we)
    assert (out.cpu().reshape(1, 240, 14, 14) - want).abs().max() < 2e-5       # NCHW memory under the declared shape


def test_bad_arguments():
    from souffle_models_b200 import efficientnet
    x, wr, we = _case(1, 7, 7, 16, 4, 1)
    with pytest.raises(ValueError):
        efficientnet.se_module(x.cuda().half(), wr.cuda(), we.cuda())
    with pytest.raises(ValueError):
        efficientnet.se_module(x.cuda(), we.cuda(), wr.cuda())
    with pytest.raises(Exception):
        efficientnet.se_module(x.cuda(), torch.zeros(80, 16).cuda(), torch.zeros(16, 80).cuda())      # reduce > 64
