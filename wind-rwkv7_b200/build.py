"""Builds lib/libwkv7_sm100.so from csrc/*.cu with nvcc for sm_100a (cross-compiles without a GPU).

    python wind-rwkv7_b200/build.py [--force] [--verbose]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OBJ = os.path.join(HERE, 'build')
LIB = os.path.join(HERE, 'lib', 'libwkv7_sm100.so')
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
         '-Xcompiler', '-fPIC', '-Xptxas', '-v']


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith('.cu'))


def _deps():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, '..', 'include', 'wkv7_sm100.h')]


def _check_tc_launch_registers(log):
    """The 4-group tcgen05 forward redistributes registers between its warp groups with setmaxnreg, whose
    blocking form waits without a bound for registers that must come out of the CTA's launch allocation.
    The kernel's arithmetic assumes that allocation is 96 registers per thread; stop the build if ptxas
    chose anything else for those instantiations."""
    lines = log.splitlines()
    seen = 0
    for i, ln in enumerate(lines):
        if 'Compiling entry function' in ln and 'wkv7_fwd_tc_kernelILi4E' in ln:
            used = next((l for l in lines[i + 1:i + 6] if 'Used' in l and 'registers' in l), '')
            seen += 1
            if 'Used 96 registers' not in used:
                raise RuntimeError('wkv7_fwd_tc_kernel<4,*> must be launched with 96 registers per thread '
                                   f'(setmaxnreg arithmetic); ptxas reports: {used.strip()!r}')
    if seen < 8:
        raise RuntimeError('ptxas log holds fewer wkv7_fwd_tc_kernel<4,*> entries than are built: cannot check their register count')


def build(force=False, verbose=False):
    newest = max(os.path.getmtime(p) for p in _deps())
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= newest:
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)

    def compile_one(src):
        obj = os.path.join(OBJ, src[:-3] + '.o')
        r = subprocess.run([NVCC] + FLAGS + ['-c', os.path.join(CSRC, src), '-o', obj],
                           capture_output=True, text=True)
        with open(os.path.join(OBJ, src[:-3] + '.ptxas.log'), 'w') as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}:\n{r.stdout}\n{r.stderr}')
        if verbose:
            print(r.stderr)
        if src == 'wkv7_fwd_tc.cu':
            _check_tc_launch_registers(r.stdout + r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, _sources()))
    # cudart is linked statically (nvcc's default): the library then does not depend on which
    # libcudart.so the host process has loaded; both attach to the device's primary context.
    subprocess.check_call([NVCC, '-gencode', 'arch=compute_100a,code=sm_100a', '-shared', '-o', LIB] + objs)
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
