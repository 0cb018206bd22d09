"""B200-native (sm_100a) build of the Distributed-HipKittens multi-GPU hot path.

The directory name carries a hyphen, so the package is loaded by path (see `load_package` in the
repository's `__graft_entry__.py`) under the module name `distributed_hipkittens_b200`.

  capi        ctypes binding of libdk_b200.so, the C ABI in include/dk_b200.h
  build       in-tree build of the library and of the pybind11 modules `iris_py` / `tk_kernel`
  torch_ops   torch.library operators (torch.ops.dk_b200.*) over the tk_kernel entry points; imported on demand
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
