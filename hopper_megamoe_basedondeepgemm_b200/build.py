"""Ahead-of-time build of the CUDA library for sm_100a (in-tree shared object, no JIT cache)."""
import os
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, 'csrc')
LIB_NAME = 'libmegamoe_b200.so'
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
# test build: the same library plus the CUDA-core cross-check engine (`engine='check'`), loaded by the tests only
CHECK_LIB_PATH = os.path.join(PKG_DIR, 'libmegamoe_b200_check.so')
SOURCES = ['mm_abi.cu']
HEADERS = ['mm_kernel.cuh', 'mm_frontend.cuh', 'mm_ptx.cuh', 'mm_prep.cuh', os.path.join('..', '..', 'include', 'megamoe_b200.h')]


def _stale(path: str) -> bool:
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, check: bool = False) -> str:
    """Compile `csrc/*.cu` into `libmegamoe_b200.so` next to this file (`check`: the test build with the cross-check
    engine, `libmegamoe_b200_check.so`); returns its path."""
    path = CHECK_LIB_PATH if check else LIB_PATH
    if not force and not _stale(path):
        return path
    nvcc = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
    cmd = [nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
           '-shared', '-Xcompiler', '-fPIC', '-o', path] + (['-DMM_WITH_CHECK_ENGINE'] if check else []) + \
          [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f'nvcc failed:\n{res.stdout}\n{res.stderr}')
    if verbose:
        print(res.stderr)
    return path


if __name__ == '__main__':
    print(build(force=True, verbose=True))
