"""Operator API, same names as the reference's flash_dropout/functional/__init__.py:1-9."""
from .blockwise_dropout_matmul_cuda import blockwise_dropout_matmul as cuda_blockwise_dropout_matmul
from .blockwise_dropout_conv2d import blockwise_dropout_conv2d as cuda_blockwise_dropout_conv2d
from .im2col_conv2d import im2col_conv2d
from .naive import blockwise_dropout_matmul as naive_blockwise_dropout_matmul
from .vanilla import dropout_matmul as vanilla_dropout_matmul

# The reference also exports a Triton twin of the CUDA op.  This engine has a single backend, so the
# name is kept and resolves to the same sm_100a kernels.
triton_blockwise_dropout_matmul = cuda_blockwise_dropout_matmul
