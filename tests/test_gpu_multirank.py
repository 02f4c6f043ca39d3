"""Expert-parallel runs over several GPUs of one node (skipped with fewer than two GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, fmt, engine='umma', mode='routed', tokens=None, window='symm_mem'):
    env = dict(os.environ, MP_FORMAT=fmt, MP_ENGINE=engine, MP_MODE=mode, MP_WINDOW=window)
    if tokens:
        env['MP_TOKENS'] = str(tokens)
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={nproc}',
           '--master-addr', '127.0.0.1', '--master-port', '29531', os.path.join(ROOT, 'tests', 'mp_worker.py')]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert 'MP_OK' in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4', 'fp8'])
def test_two_ranks(fmt):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    _run(2, fmt)


def test_two_ranks_over_the_librarys_own_window():
    """The buffer allocated and mapped through mm_window_alloc / mm_window_open (inter-process memory handles gathered
    once over the NCCL group) instead of torch's symmetric memory."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    _run(2, 'mxfp4', window='ipc')


def test_two_ranks_many_tokens():
    """48 and 45 tokens x top-4: ~96 rows per destination, so several SMs share each dispatch."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    _run(2, 'mxfp4', tokens=48)


def test_two_ranks_from_hidden_states():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    _run(2, 'mxfp4', mode='from_hidden')


def test_skewed_routing_from_hidden_states_on_all_gpus():
    """Sigmoid scores + Zipf(1.2) expert bias over all ranks' experts, 16 tokens per rank, router fused into the launch:
    hot experts receive more than 16 rows from several source ranks (32-row token tiles), counts and top-8 exact."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs two GPUs')
    _run(8 if n >= 8 else (4 if n >= 4 else 2), 'mxfp4', mode='from_hidden_skewed')


def test_all_ranks_of_the_node():
    n = torch.cuda.device_count()
    if n < 4:
        pytest.skip('needs at least four GPUs')
    _run(8 if n >= 8 else 4, 'mxfp4')


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4', 'fp8'])
def test_full_shape_parity_on_all_gpus(fmt):
    """The benchmark's own configuration (48 experts per rank, H=3072, I=1280, top-8, forced-balanced routing) on every
    GPU of the node: the benchmark checks its output, counts and slot maps against the oracle and reports `parity`."""
    import json
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs two GPUs')
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={n}', '--master-addr', '127.0.0.1',
           '--master-port', '29533', os.path.join(ROOT, 'bench.py'), '--gpus', str(n), '--steps', '5', '--warmup', '3',
           '--format', fmt, '--no-cpu-baseline'] + (['--no-sweep'] if fmt != 'mxfp4' else [])
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith('{')]
    assert res.returncode == 0 and lines, res.stdout[-3000:] + res.stderr[-3000:]
    out = json.loads(lines[-1])
    assert out['parity']['ok'] and out['parity']['slot_map_exact'] and out['parity']['counts_exact'], out['parity']
    if 'm_sweep' in out:
        assert all(v['parity_ok'] for v in out['m_sweep'].values()), out['m_sweep']
