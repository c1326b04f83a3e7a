"""Compile libbongard_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / 'csrc'
LIB = HERE / 'libbongard_b200.so'
SOURCES = ['api.cu', 'glue.cu', 'glue_bwd.cu', 'gemm_bf16.cu', 'gemm_bf16_pair.cu', 'gemm_bf16_skinny.cu', 'gemm_fp8.cu', 'gemm_mxfp8.cu', 'attn.cu', 'attn_pair.cu', 'attn_bwd.cu']
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
         '-Xcompiler', '-fPIC', '-cudart', 'static']


def nvcc():
    for candidate in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if candidate and (candidate == 'nvcc' or Path(candidate).exists()):
            return candidate
    raise RuntimeError('nvcc not found')


def stale():
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    return any(p.stat().st_mtime > built for p in list(CSRC.glob('*.cu')) + list(CSRC.glob('*.cuh')))


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    objects = []
    build_dir = HERE / 'build'
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = build_dir / (src + '.o')
        objects.append(str(obj))
        cmd = [nvcc(), *FLAGS, '-c', str(CSRC / src), '-o', str(obj)]
        if verbose:
            cmd.insert(1, '-Xptxas')
            cmd.insert(2, '-v')
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode or verbose:
            print(f'--- {src}\n{out}', file=sys.stderr)
        failed |= bool(proc.returncode)
    if failed:
        raise RuntimeError('nvcc failed')
    subprocess.check_call([nvcc(), '-shared', '-cudart', 'static', '-o', str(LIB), *objects])
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
