"""Import-name shim: `import bert_binding` resolves here when this directory is on sys.path,
as the reference's callers expect (cpp/bert/bert_binding.cu:537-540; used by
python/models/bert/souffle_bert.py:9-17 and cpp/bert/test_bert_binding.py)."""
from souffle_models_b200.bert import souffle_bert_layer  # noqa: F401
