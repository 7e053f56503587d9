"""Import-name shim for lstm_binding.fused_lstm (cpp/lstm/lstm_binding.cu:75-78; called by
python/models/lstm/souffle_lstm.py:184-197 and cpp/lstm/test_lstm.py)."""
from souffle_models_b200.lstm import fused_lstm  # noqa: F401
