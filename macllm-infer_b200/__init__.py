"""macllm_b200: the B200-native continuous-batching step of macllm-infer.

The directory name carries a hyphen, so the package is imported under the name ``macllm_infer_b200``
through :func:`__graft_entry__.load_package` (or any importlib call that gives it that name).

Submodules
  _capi    ctypes binding of libmacllm_b200.so (C ABI in include/macllm_b200.h)
  ops      NumPy wrappers of the kernel-level entry points
  kv       host-only paged-KV pool / block tables / prefix cache (mirrors crates/macllm-kv)
  model    CausalLm-shaped model / session / reservation objects
  engine   the continuous-batching engine (ServingScheduler-shaped)
  seed_gguf  synthetic GGUF checkpoint writer for the benchmark configurations
  build    nvcc build of the shared library
"""
from . import _capi  # noqa: F401

__all__ = ["_capi"]
