"""In-tree build of the sm_100a shared library (``libadacode_sm100.so``).

``python -m adacode_b200.build`` compiles ``csrc/*.cu`` with nvcc for ``sm_100a`` only.
nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT_DIR = os.path.dirname(PKG_DIR)
LIB_PATH = os.path.join(PKG_DIR, 'libadacode_sm100.so')
NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
    '-Xcompiler', '-fPIC', '-shared',
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(PKG_DIR, 'csrc', '*.cu')))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(ROOT_DIR, 'include', '*.h')) + glob.glob(os.path.join(PKG_DIR, 'csrc', '*.cuh'))
    return any(os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get('NVCC', 'nvcc')
    cmd = [nvcc, *NVCC_FLAGS, '-I', os.path.join(ROOT_DIR, 'include'), '-o', LIB_PATH, *sources()]
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f'nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}')
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
