"""Import-name shim for efficientnet_se_module_binding (cpp/efficientnet/efficientnet_se_module_binding.cu:229-233)."""
from souffle_models_b200.efficientnet import torch_dispatch_efficientnet_se_module_v2_short_cut_fused  # noqa: F401
