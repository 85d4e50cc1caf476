"""Loader of the native module.  Import fails loudly when the module is absent: there is no
Python fallback for the executor."""
import importlib.util
import os

from msccl.runtime.build import MODULE, module_path

_module = None


class NativeRuntimeMissing(ImportError):
    pass


def load(build_if_missing=False):
    global _module
    if _module is not None:
        return _module
    path = module_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise NativeRuntimeMissing(
                f'{path} is missing: run "python -m msccl.runtime.build" (needs nvcc) before using msccl.runtime')
        from msccl.runtime.build import build
        build()
    spec = importlib.util.spec_from_file_location(f'msccl.runtime.{MODULE}', path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _module = mod
    return mod
