"""souffle_models_b200: B200-native (sm_100a) fused global-sync encoder kernels behind the
reference's binding names.  The compute lives in lib/libsouffle_b200.so (C ABI in
include/souffle_b200.h); this package is the thin host-side mirror of the reference's
Python-facing interface."""
from ._lib import SouffleError, load  # noqa: F401
