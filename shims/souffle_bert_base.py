"""Import-name shim for souffle_bert_base.souffle_bert_base (cpp/bert/bert_base_impl.cu:277-308, 1783-1786;
imported by python/models/bert/souffle_bert.py:5 for opt level O0)."""
from souffle_models_b200.bert import souffle_bert_base  # noqa: F401
