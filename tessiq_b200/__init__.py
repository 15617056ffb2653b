"""tessiq_b200 — a B200 (sm_100a) kernel layer for tessiq's data-parallel hot path.

    tessiq_b200.kernel   the `Kernel` launch interface (FusedKernel, ReductionKernel, PackKernel, …)
    tessiq_b200.ops      eager entry points and the `torch.ops.tessiq.<name>` custom operations
    tessiq_b200.build    builds libtessiq_b200.so in tree (`python -m tessiq_b200.build`)

Submodules load on first use so that `python -m tessiq_b200.build` works before the library
exists. There is no CPU or pure-PyTorch path: using `kernel` or `ops` without the built library
raises ImportError.
"""

from importlib import import_module

__version__ = "0.1.0"
_SUBMODULES = ("kernel", "ops", "build", "backend", "executor", "sharding")


def __getattr__(name):
    if name in _SUBMODULES:
        return import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
