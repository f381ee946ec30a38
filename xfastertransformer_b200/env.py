"""``get_env()`` of the reference returns an ``LD_PRELOAD=libiomp5.so`` line for its OpenMP runtime
(``src/xfastertransformer/env.py:15-21``).  A CUDA build preloads nothing; the function is kept so
launch scripts of the form ``$(python -c 'import xfastertransformer as xft; print(xft.get_env())')``
still work, and returns the NCCL settings this engine recommends on NVSwitch systems."""


def get_env() -> str:
    return "NCCL_NVLS_ENABLE=1 CUDA_DEVICE_MAX_CONNECTIONS=1"
