"""The standalone hardware microbenchmarks under fly_b200/microbench must keep compiling for sm_100a against the
kernels' own PTX helpers (nvcc cross-compiles; nothing is run here)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = os.environ.get('NVCC') or shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'


@pytest.mark.skipif(not os.path.exists(NVCC), reason='nvcc not found')
@pytest.mark.parametrize('name', ['mma_cost', 'tma_ring'])
def test_microbench_compiles(name, tmp_path):
    src = os.path.join(ROOT, 'fly_b200', 'microbench', name + '.cu')
    cmd = [NVCC, '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17',
           '-I', os.path.join(ROOT, 'fly_b200', 'csrc'), '-I', os.path.join(ROOT, 'include'),
           '-c', src, '-o', str(tmp_path / (name + '.o'))]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
