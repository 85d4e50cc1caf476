"""Build the native runtime (``csrc/`` -> ``msccl/runtime/_msccl_native*.so``) with nvcc for sm_100a.

The shared object is kept inside the package so that it travels with the source tree; nothing is
installed into site-packages.  ``python -m msccl.runtime.build`` rebuilds it.
"""
import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CSRC = os.path.join(ROOT, 'csrc')
MODULE = '_msccl_native'
ARCH_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a']
SOURCES = ['exec_kernel.cu', 'direct_kernels.cu', 'gemm_sm100.cu', 'gemm_2cta_sm100.cu', 'gemm_mxfp8_sm100.cu', 'gemm_mxfp8_2cta_sm100.cu', 'fused_tp.cu', 'fused_tp_2cta.cu', 'fused_tp_fp8.cu', 'fused_tp_fp8_2cta.cu', 'quantize_mx.cu', 'moe_a2a.cu', 'moe_a2a_2cta.cu', 'moe_route.cu', 'no_alloc.cu',
           'symm_mem.cpp', 'bindings.cpp']


def _nvcc():
    for cand in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError('nvcc not found')


def module_path():
    suffix = sysconfig.get_config_var('EXT_SUFFIX') or '.so'
    return os.path.join(HERE, MODULE + suffix)


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def source_digest():
    h = hashlib.sha256()
    for path in sorted(_sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.h', '.cuh'))]):
        with open(path, 'rb') as f:
            h.update(path.encode() + b'\0' + f.read())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compile every source for sm_100a and link the Python module.  Returns the module path."""
    import pybind11
    out = module_path()
    stamp = out + '.digest'
    digest = source_digest()
    if not force and os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == digest:
        return out
    obj_dir = os.path.join(HERE, '_obj')
    os.makedirs(obj_dir, exist_ok=True)
    include = ['-I', CSRC, '-I', pybind11.get_include(), '-I', sysconfig.get_paths()['include']]
    common = ['-std=c++17', '-O3', '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden', '-lineinfo']
    objects = []
    procs = []
    for src in _sources():
        obj = os.path.join(obj_dir, os.path.basename(src) + '.o')
        cmd = [_nvcc()] + ARCH_FLAGS + common + include + ['-c', src, '-o', obj]
        if verbose:
            cmd.insert(1, '-Xptxas=-v')
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(obj)
    for src, proc in procs:
        text, _ = proc.communicate()
        if verbose and text:
            print(text)
        if proc.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}:\n{text}')
    link = [_nvcc()] + ARCH_FLAGS + ['-shared', '-Xcompiler', '-fPIC', '-o', out] + objects + ['-cudart', 'static']
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError(f'link failed:\n{done.stdout}')
    with open(stamp, 'w') as f:
        f.write(digest)
    return out


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
