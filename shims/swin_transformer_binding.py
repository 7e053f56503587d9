"""Import-name shim for swin_transformer_binding (cpp/swin_transformer/swin_transformer_binding.cu:276-289;
called by python/models/swin_transformer/swin_mlp.py:29,338-339).  `swin_stage` is an addition: a chain of blocks and
the patch merging after them as one launch."""
from souffle_models_b200.swin import (bench_swin_ffn, bench_swin_fused_feed_mlp, swin_ffn,  # noqa: F401
                                      swin_fused_feed_mlp, swin_stage)
