"""b200mono: B200 (sm_100a) persistent decode monokernels behind the sgl-amd-mono plugin surface.

Layout
  csrc/      CUDA kernels and the C ABI (``include/b200mono.h``), built by ``build.py``
  cabi.py    ctypes view of the C ABI (structs parsed from the header)
  ffn.py     host runner of the MoE FFN launch
There is no CPU or PyTorch fallback: the kernels run through ``libb200mono.so`` or not at all.
"""

__version__ = "0.1.0"
BACKEND = "b200"
