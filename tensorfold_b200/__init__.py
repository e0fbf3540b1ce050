"""B200-native kernels behind TensorFold's quantized-projection entry points (affine packed-row matmul, MoE experts,
tensor-parallel linears).  Python here is plumbing: it validates arguments, owns no arithmetic, and calls the CUDA
library through its C ABI (``include/tensorfold_b200.h``).  There is no CPU fallback."""

__version__ = "0.1.0"
