"""B200-native Multi-head Latent Attention behind the dscuda host API.

`dscuda_b200.build` compiles the CUDA sources (sm_100a only) into
`build/libdscuda_mla_bench.so` and `build/libdscuda_flash_attention_bench.so`;
`dscuda_b200.mla` is the Python host side that calls them through ctypes the way
the reference's `benchmarks/mla.py` does.  There is no CPU or PyTorch fallback:
if the libraries are missing or no GPU is present, calls raise.
"""

from . import build, library  # noqa: F401
