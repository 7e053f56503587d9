"""Import-name shim for swin_trans_fc2.swin_trans_fc2 (cpp/swin_transformer/swin_trans_fc2_binding.cu:58-61)."""
from souffle_models_b200.swin import swin_trans_fc2  # noqa: F401
