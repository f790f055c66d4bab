"""B200-native SparseDrop: the ``flash_dropout`` operator and module API on sm_100a kernels."""


def check_status(device=None) -> None:
    """Failure detection for the CUDA kernels: raises if a launch on ``device`` (default: the current one) gave up
    on a bounded device-side wait since the last check.  See ``flash_dropout.cuda.binding_gemm.check_status``."""
    from flash_dropout.cuda.binding_gemm import check_status as _check
    _check(device)


def set_sm_margin(sms: int) -> int:
    """SMs that every later GEMM / conv launch leaves free for a kernel running beside it (a gradient all-reduce
    that overlaps the next step's products); returns the previous value.  0 (the default) uses every SM."""
    from flash_dropout import _lib
    prev = _lib.lib().sd_set_sm_margin(int(sms))
    _lib.check(min(prev, 0))
    return prev
