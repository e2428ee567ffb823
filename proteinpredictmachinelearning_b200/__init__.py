"""B200-native dense-contraction kernels behind the PPML graph executor's per-op launcher API.

The product is libppml_b200.so (C ABI in include/ppml_b200.h, C++ forwarders under the
reference's own launcher names).  This package is the Python host-side mirror of that interface
used by the tests and the benchmark; torch only provides device memory and streams."""
from ._lib import LIB_PATH, PATH_AUTO, PATH_SIMT, PATH_UMMA, TF32_ROUND, TF32_TMA, TF32_TRUNCATE, load  # noqa: F401
