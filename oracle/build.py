"""Compile the CPU oracle (oracle/tkq_oracle.c) into oracle/libtkq_oracle.so.

Test infrastructure only: the product never loads this library.

Flags that matter for bit-exactness with the CUDA kernels:
  -ffp-contract=off   a*b+c is never fused behind the source's back; fused
                      multiply-adds happen only where the source calls fmaf()
  (no -ffast-math)    IEEE division, no flush-to-zero, no reassociation
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, 'tkq_oracle.c')
LIB = os.path.join(HERE, 'libtkq_oracle.so')


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ['gcc', '-O3', '-std=c11', '-fopenmp', '-ffp-contract=off', '-mavx2', '-mfma', '-fPIC', '-shared',
           SRC, '-o', LIB, '-lm']
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv))
