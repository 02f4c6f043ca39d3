"""Ahead-of-time build of the CUDA library for sm_100a (in-tree shared object, no JIT cache)."""
import os
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, 'csrc')
LIB_NAME = 'libmegamoe_b200.so'
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
SOURCES = ['mm_abi.cu']
HEADERS = ['mm_kernel.cuh', 'mm_frontend.cuh', 'mm_ptx.cuh', 'mm_prep.cuh', os.path.join('..', '..', 'include', 'megamoe_b200.h')]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile `csrc/*.cu` into `libmegamoe_b200.so` next to this file; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
    cmd = [nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
           '-shared', '-Xcompiler', '-fPIC', '-o', LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f'nvcc failed:\n{res.stdout}\n{res.stderr}')
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force=True, verbose=True))
