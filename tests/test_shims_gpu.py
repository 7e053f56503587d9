"""The reference's caller scripts against the import-name shims.

The reference's own scripts (cpp/lstm/test_lstm.py:5-14, cpp/bert/test_bert_binding.py:7-15,
cpp/swin_transformer/test_swin_transformer_binding.py:20-36, 39-47, 50-56) import the binding modules by name
and call them positionally.  Each case below is a fresh interpreter with only `shims/` and the repository root on
its path that makes the same imports and the same calls, with the same argument shapes, dtypes and order, and
prints what the script prints; on top of that the result is checked (shape, dtype, finite, and the value where the
inputs make one easy to state).  The reference checkout itself is not read.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LSTM_CALLER = r"""
import torch
import lstm_binding

batch_size, num_layer, num_hidden, num_timestep = 1, 10, 256, 100
input_timestep = torch.ones((batch_size, num_timestep, num_hidden), dtype=torch.float32, device="cuda")
weight_input_wavefront = torch.ones((4 * num_layer, num_hidden, num_hidden), dtype=torch.float32, device="cuda")
weight_state_wavefront = torch.ones((4 * num_layer, num_hidden, num_hidden), dtype=torch.float32, device="cuda")
output_timestep = lstm_binding.fused_lstm(input_timestep, weight_input_wavefront, weight_state_wavefront)
print(output_timestep)
assert output_timestep.shape == (1, 100, 256) and output_timestep.dtype == torch.float32 and output_timestep.is_cuda
assert torch.isfinite(output_timestep).all()
# all-ones weights saturate every gate: the first output row is the zero-input response of the stack (inputs arrive
# one step late, cpp/lstm/lstm_reuse_shared_memory.cu:324-326), later rows approach tanh(c) with c growing by ~1 a step
assert output_timestep[0, 0].abs().max() < 0.5 and output_timestep[0, -1].min() > 0.99
print("LSTM_OK")
"""

BERT_CALLER = r"""
import torch
import bert_binding

batch_size, num_heads, max_seq_length, num_hidden, d_intermedia = 1, 12, 384, 64, 3072
hidden_size = num_heads * num_hidden
torch.manual_seed(0)
for opt_level in (3, 4):
    src = torch.randn(batch_size, max_seq_length, hidden_size).to(torch.float16).to('cuda')
    qkv_weight = torch.randn(3, hidden_size, hidden_size).to(torch.float16).to('cuda')
    attn_fc_weight = torch.randn(hidden_size, hidden_size).to(torch.float16).to('cuda')
    feed_forward_fc1_weight = torch.randn(hidden_size, d_intermedia).to(torch.float16).to('cuda')
    feed_forward_fc2_weight = torch.randn(d_intermedia, hidden_size).to(torch.float16).to('cuda')
    output = bert_binding.souffle_bert_layer(src, qkv_weight, attn_fc_weight, feed_forward_fc1_weight,
                                             feed_forward_fc2_weight, opt_level)
    print(output[-1])
    assert [tuple(t.shape) for t in output] == [(3, 12, 384, 64), (12, 384, 384), (384, 768), (384, 768), (384, 3072), (384, 768)]
    assert all(t.dtype == torch.float16 and t.is_cuda for t in output)
    # unit-variance weights overflow fp16 inside the reference too; the two LayerNorm outputs and the probabilities
    # are the tensors that stay finite whatever the scale
    assert torch.isfinite(output[1].float()).all() and (output[1].float().sum(-1) - 1).abs().max() < 2e-2
    assert torch.isfinite(output[3].float()).all()
print("BERT_OK")
"""

SWIN_CALLER = r"""
import torch
import swin_transformer_binding
import swin_trans_fc2

torch.manual_seed(0)
batch_size, seq_length, in_features, out_features = 1, 256, 512, 2048
src = torch.rand((batch_size * seq_length, in_features), dtype=torch.half, device="cuda").uniform_(-1, 1) / 16
fc1_weight = (torch.rand((in_features, out_features), device="cuda").uniform_(-1, 1) / 16).to(torch.float16)
fc2_weight = (torch.rand((out_features, in_features), device="cuda").uniform_(-1, 1) / 16).to(torch.float16)
fc1_output, fc2_output = swin_transformer_binding.swin_fused_feed_mlp(src, fc1_weight, fc2_weight)
print(fc2_output)
assert fc1_output.shape == (256, 2048) and fc2_output.shape == (256, 512)
want1 = src.float() @ fc1_weight.float()
assert (fc1_output.float() - want1).abs().max() < 2e-3
assert (fc2_output.float() - fc1_output.float() @ fc2_weight.float()).abs().max() < 4e-3

M, N, K = 256, 2048, 512
src = torch.rand((M, K), dtype=torch.half, device="cuda").uniform_(-1, 1) / 16
w1 = torch.randn((K, N), dtype=torch.half, device="cuda").uniform_(-1, 1) / 16
w2 = torch.randn((N, K), dtype=torch.half, device="cuda").uniform_(-1, 1) / 16
o1 = swin_transformer_binding.swin_ffn(src, w1, M, N, K)
print(o1.shape)
o2 = swin_transformer_binding.swin_ffn(o1, w2, M, K, N)
print(o2)
assert o1.shape == (M, N) and o2.shape == (M, K)
assert (o2.float() - o1.float() @ w2.float()).abs().max() < 4e-3

latency = swin_transformer_binding.bench_swin_fused_feed_mlp(src, fc1_weight, fc2_weight, 1, 1, 1)
print(latency)
assert isinstance(latency, float) and 0 < latency < 1e5
latency = swin_transformer_binding.bench_swin_ffn(M, K, N, 10, 3, 100)
assert isinstance(latency, float) and 0 < latency < 1e5

M, N, K = 256, 512, 2048
src = torch.ones((1, M, K), dtype=torch.half, device="cuda") / 16
weight = torch.ones((K, N), dtype=torch.half, device="cuda") / 16
output = swin_trans_fc2.swin_trans_fc2(src, weight)
print(output)
assert output.shape == (1, M, N) and (output.float() - K / 256.0).abs().max() < 1e-2
print("SWIN_OK")
"""


def _run(script: str, marker: str) -> None:
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "shims"), ROOT])
    res = subprocess.run([sys.executable, "-c", script], env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert marker in res.stdout


def test_lstm_caller_runs_against_the_shim():
    _run(LSTM_CALLER, "LSTM_OK")


def test_bert_caller_runs_against_the_shim():
    _run(BERT_CALLER, "BERT_OK")


def test_swin_callers_run_against_the_shims():
    _run(SWIN_CALLER, "SWIN_OK")
