"""B200-native SparseDrop: the ``flash_dropout`` operator and module API on sm_100a kernels."""
