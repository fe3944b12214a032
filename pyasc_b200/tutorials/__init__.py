"""asc2 kernels for the B200 workloads, written the way the reference writes its asc2 kernel
tests (python/test/asc2/kernels/*.py): an ``@asc2.jit`` kernel plus a ``*_launch`` helper that picks
``core_num`` and tile sizes.  The vector-add and softmax kernels are the reference's own forms; the
K-looped fp16 GEMM, the int8 GEMM and attention are new scripts in the same style (the reference has
no asc2 kernel for them); GELU and leaky ReLU are the reference's elementwise kernel tests."""
from .vadd import vadd_kernel, vadd_launch  # noqa: F401
from .softmax import softmax_kernel, softmax_launch, softmax_fused_kernel, softmax_fused_launch  # noqa: F401
from .matmul_fp16 import matmul_fp16_kernel, matmul_fp16_launch  # noqa: F401
from .matmul_int8 import (matmul_int8_kernel, matmul_int8_launch, matmul_int8_dequant_kernel,  # noqa: F401
                          matmul_int8_dequant_launch)
from .flash_attention import attention_kernel, attention_launch  # noqa: F401
from .gelu import gelu_kernel, gelu_launch  # noqa: F401
from .leaky_relu import leaky_relu_kernel, leaky_relu_launch  # noqa: F401
