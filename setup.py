"""Packaging: ``pip install -e .`` (or ``python setup.py build_ext --inplace``) compiles the native module
for sm_100a with nvcc into ``msccl/runtime/`` and installs the ``msccl`` command.

The Python tool stack (DSL, synthesis, CLI, CPU interpreter) works without the native module; the build
step is skipped with a note when nvcc is not available.
"""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

HERE = os.path.dirname(os.path.abspath(__file__))


def compile_native():
    sys.path.insert(0, HERE)
    try:
        from msccl.runtime.build import build
        print('msccl: native module at', build())
    except Exception as e:      # noqa: BLE001 - the pure-Python parts remain usable
        print(f'msccl: native module not built ({type(e).__name__}: {e}); the executor and the GPU ops need it')
    finally:
        sys.path.remove(HERE)


class BuildNative(Command):
    description = 'compile csrc/ for sm_100a into msccl/runtime/ (nvcc)'
    user_options = [('inplace', 'i', 'accepted for compatibility; the module is always built in tree')]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        compile_native()


class BuildPyWithNative(build_py):
    def run(self):
        compile_native()
        super().run()


class DevelopWithNative(develop):
    def run(self):
        compile_native()
        super().run()


setup(
    name='msccl-b200',
    version='0.1.0',
    description='MSCCLang, collective synthesis and a native B200 executor with fused compute+collective kernels',
    packages=find_packages(include=['msccl', 'msccl.*']),
    package_data={'msccl.autosynth': ['msccl_ndv2_launcher.sh'], 'msccl.runtime': ['_msccl_native*.so', '*.digest']},
    scripts=['msccl/autosynth/msccl_ndv2_launcher.sh'],
    entry_points={'console_scripts': ['msccl = msccl.__main__:main']},
    python_requires='>=3.10',
    install_requires=['z3-solver', 'tabulate', 'torch'],
    extras_require={'completion': ['argcomplete']},
    cmdclass={'build_ext': BuildNative, 'build_py': BuildPyWithNative, 'develop': DevelopWithNative},
)
