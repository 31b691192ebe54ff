"""Build libtkquant.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m tilekernels_b200.build [--force] [--verbose]

Flags that matter for results:
  -fmad=false     multiplications and additions are never contracted into FMAs
                  behind the source's back; the kernels call fmaf explicitly
                  where a fused operation is part of the algorithm
  (no --use_fast_math)  IEEE division, no flush-to-zero
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
INCLUDE = os.path.join(os.path.dirname(HERE), 'include')
LIB_DIR = os.path.join(HERE, 'lib')
LIB = os.path.join(LIB_DIR, 'libtkquant.so')
SOURCES = ['tkq_api.cu', 'tkq_per_token.cu', 'tkq_swiglu.cu', 'tkq_tile.cu', 'tkq_cast_back.cu', 'tkq_swiglu_backward.cu', 'tkq_expand.cu']
NVCC_FLAGS = ['-O3', '-std=c++17', '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-fmad=false',
              '-Xcompiler', '-fPIC', '-I' + INCLUDE, '-I' + CSRC]


def _newest_source_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, 'tkquant.h')]
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime():
        return LIB
    nvcc = os.environ.get('NVCC', 'nvcc')
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIB_DIR, src.replace('.cu', '.o'))
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-c', os.path.join(CSRC, src), '-o', obj]
        procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, proc in procs:
        if proc.wait() != 0:
            raise RuntimeError('nvcc failed: ' + ' '.join(cmd))
    subprocess.run([nvcc, '-shared', '-o', LIB] + objs, check=True)
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
