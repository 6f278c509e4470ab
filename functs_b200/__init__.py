"""functs_b200: B200 (sm_100a) executor for the fusion groups that FuncTs' TensorSSA functionalization produces.

The package has three layers:
  * ``libfuncts_b200.so`` — hand-written CUDA kernels behind a C ABI (include/functs_b200.h);
  * ``functs_b200.ops`` / ``functs_b200.immut`` — tensor-level wrappers (torch owns memory and streams);
  * ``functs_b200.workloads`` — mirrors of the reference's post-processing modules.
Importing the package loads the shared library and raises if it is missing: there is no CPU fallback.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is absent)
from . import access_desc, immut, ops, workloads  # noqa: F401
from ._lib import FunctsB200Error, launch_count  # noqa: F401

__all__ = ["access_desc", "immut", "ops", "workloads", "FunctsB200Error", "launch_count"]
