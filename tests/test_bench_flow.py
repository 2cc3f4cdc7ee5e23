"""Control flow of bench.py's 8-GPU default run, on CPU with the measurement replaced by a stand-in: the main line is
printed exactly once whatever becomes of the extra 1.5D measurement (result, exception, no answer before the deadline)."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

DRIVER = r'''
import json, os, sys, time
sys.path.insert(0, {root!r})
os.environ.update(RANK='0', WORLD_SIZE='8')
import torch
torch.cuda.is_available = lambda: True
import bench
mode = sys.argv[1]
bench.CONFIG3_DEADLINE_S = 1 if mode == 'stuck' else 60
calls = []

def fake_measure(args, rank, world, keep_process_group=False):
    calls.append((args.rep, args.layers, keep_process_group))
    if len(calls) == 2:
        if mode == 'raises':
            raise RuntimeError('second layout failed')
        if mode == 'stuck':
            time.sleep(20)
    line = dict(metric='gcn_epoch_ms', value=15.7 if args.rep == 1 else 33.6, unit='ms', steps=2, warmup=3, config=dict(rep=args.rep),
                run=dict(stage_order='x'), parity=dict(ok=mode != 'bad_parity' or args.rep == 1, max_rel=1e-8), e2e=dict(value=1.0),
                roofline=dict(achieved=1.0, peak=2.0, unit='GB/s', frac=0.5, spmm_ms_per_step=1.0, products_per_step=8, kernel='k'))
    return line, line['parity']['ok']

bench.measure = fake_measure
sys.argv = ['bench.py', '--gpus', '8'] + sys.argv[2:]
bench.run_ours(bench.parse())
print('calls', calls)
'''


def _run(mode, *flags):
    out = subprocess.run([sys.executable, '-c', DRIVER.format(root=ROOT), mode, *flags], capture_output=True, text=True, timeout=120)
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith('{')]
    return out, lines


def test_default_8_gpu_run_appends_the_15d_configuration():
    out, lines = _run('fine')
    assert out.returncode == 0, out.stderr
    assert len(lines) == 1 and lines[0]['value'] == 15.7
    extra = lines[0]['config3']
    assert extra['value'] == 33.6 and extra['config'] == {'rep': 2} and extra['parity']['ok'] and extra['roofline']['frac'] == 0.5
    assert "calls [(1, 0, True), (2, 4, False)]" in out.stdout


def test_workload_flags_switch_the_extra_measurement_off():
    for flags in (('--no-config3',), ('--rep', '2'), ('--stage-group', '1'), ('--config', 'dense233k')):
        out, lines = _run('fine', *flags)
        assert out.returncode == 0, out.stderr
        assert len(lines) == 1 and 'config3' not in lines[0]
        assert out.stdout.count('False)]') == 1 and '), (' not in out.stdout.split('calls')[-1]


@pytest.mark.parametrize('mode,note', [('raises', 'second layout failed'), ('stuck', 'no result within 1 s')])
def test_main_line_survives_a_failed_extra_measurement(mode, note):
    out, lines = _run(mode)
    assert out.returncode == 0, out.stderr
    assert len(lines) == 1 and lines[0]['value'] == 15.7
    assert note in lines[0]['config3']['error']


def test_failed_parity_of_the_extra_measurement_is_loud():
    out, lines = _run('bad_parity')
    assert out.returncode != 0
    assert len(lines) == 1 and lines[0]['config3']['parity']['ok'] is False
    assert 'config3' in out.stderr
