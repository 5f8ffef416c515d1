"""B200-native GGUF-block quantized matmul (Q8_0 / Q4_K / Q6_K) behind the
nates-recipe-rs kernel-launcher convention.  The compute lives in libqmm.so
(hand-written CUDA for sm_100a, C ABI in include/qmm.h); this package is the
thin host-side mirror used by the tests and the benchmark."""
from ._lib import Q4_K, Q6_K, Q8_0, Q8_1, BLOCK_BYTES, BLOCK_ELEMS, LIB_PATH, QmmError, lib  # noqa: F401
