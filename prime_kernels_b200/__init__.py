"""Registry of the B200-native kernels.

Same public surface and behaviour as the reference registry (prime_kernels/__init__.py:12-78 in the
reference project): ``KERNELS``, ``spec``, ``is_built``, ``unavailable_reason``, ``is_available``,
``load`` and ``status``.  A kernel is available when its shared library is built, its import
requirements are present, a CUDA device exists and the device capability matches one of the
table's ``arch`` entries exactly.  There is no CPU fallback: ``load`` raises ``RuntimeError`` with
the reason instead.
"""
from __future__ import annotations

import importlib
import importlib.util
from pathlib import Path
from types import ModuleType

from ._spec import Arch, KernelSpec
from ._spec import load as _load_manifest

__all__ = ["Arch", "KernelSpec", "KERNELS", "is_available", "is_built", "load", "spec", "status",
           "unavailable_reason"]

_PACKAGE_DIR = Path(__file__).resolve().parent
_SPECS: dict[str, KernelSpec] = _load_manifest(_PACKAGE_DIR)
_LOADED: dict[str, ModuleType] = {}

KERNELS: tuple[str, ...] = tuple(_SPECS)

LIBRARY = _PACKAGE_DIR / "lib" / "libprime_kernels_b200.so"
BINDING = _PACKAGE_DIR / "lib" / "libprime_kernels_b200_torch.so"


def spec(name: str) -> KernelSpec:
    if name not in _SPECS:
        raise KeyError(f"unknown kernel {name!r}, have {', '.join(KERNELS) or '<none>'}")
    return _SPECS[name]


def is_built(name: str) -> bool:
    kernel = spec(name)
    if kernel.python_only:
        return (kernel.path / "__init__.py").is_file()
    return LIBRARY.exists() and BINDING.exists()


def unavailable_reason(name: str, device: int | None = None) -> str | None:
    import torch

    kernel = spec(name)
    if not is_built(name):
        return f"{name} was not compiled into this install of prime-kernels"
    missing = [req for req in kernel.requires if importlib.util.find_spec(req) is None]
    if missing:
        return f"{name} requires {', '.join(missing)}, which is not installed"
    if not torch.cuda.is_available():
        return f"{name} requires a CUDA device ({kernel.sm_list}), none is available"
    capability = torch.cuda.get_device_capability(device)
    if not kernel.supports(capability):
        return f"{name} requires {kernel.sm_list}, this device is sm_{capability[0]}{capability[1]}"
    return None


def is_available(name: str, device: int | None = None) -> bool:
    return unavailable_reason(name, device) is None


def load(name: str, device: int | None = None) -> ModuleType:
    try:
        return _LOADED[name]
    except KeyError:
        pass
    reason = unavailable_reason(name, device)
    if reason is not None:
        raise RuntimeError(reason)
    module = importlib.import_module(spec(name).module)
    _LOADED[name] = module
    return module


def status(device: int | None = None) -> dict[str, str]:
    return {name: unavailable_reason(name, device) or "available" for name in KERNELS}
