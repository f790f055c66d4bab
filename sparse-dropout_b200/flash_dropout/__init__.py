"""B200-native SparseDrop: the ``flash_dropout`` operator and module API on sm_100a kernels."""


def check_status(device=None) -> None:
    """Failure detection for the CUDA kernels: raises if a launch on ``device`` (default: the current one) gave up
    on a bounded device-side wait since the last check.  See ``flash_dropout.cuda.binding_gemm.check_status``."""
    from flash_dropout.cuda.binding_gemm import check_status as _check
    _check(device)
