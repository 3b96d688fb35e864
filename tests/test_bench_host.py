"""Host-side pieces of bench.py that need no GPU: the clock sampler against a stand-in nvidia-smi."""
import importlib.util
import os
import stat
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def bench():
  spec = importlib.util.spec_from_file_location('bench_under_test', os.path.join(ROOT, 'bench.py'))
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  return mod


def _fake_smi(tmp_path, body):
  path = tmp_path / 'nvidia-smi'
  path.write_text('#!/bin/sh\n' + body)
  path.chmod(path.stat().st_mode | stat.S_IXUSR)
  return str(tmp_path)


def test_clock_sampler_waits_for_the_first_line_and_keeps_sampling(bench, tmp_path, monkeypatch):
  # a sampler that needs a moment to start, then prints one line per 50 ms for GPU 3
  body = ('sleep 0.4\n'
          'while true; do echo "3, 1965, 1965, 612.3, 0x0000000000000004, Not Active, Not Active, '
          'Not Active, Active"; sleep 0.05; done\n')
  monkeypatch.setenv('PATH', _fake_smi(tmp_path, body) + os.pathsep + os.environ['PATH'])
  s = bench.ClockSampler(3)
  t0 = time.perf_counter()
  s.wait_first_sample(timeout=5.0)
  assert time.perf_counter() - t0 >= 0.4            # it did wait for the start-up
  assert s.first.startswith('3,')
  time.sleep(0.3)
  out = s.stop()
  assert out['sm_mhz'] == 1965.0 and out['sm_max_mhz'] == 1965.0
  assert out['reasons'] == ['sw_power_cap']
  assert out['samples'] >= 3                        # the first line and what followed it


def test_clock_sampler_gives_up_on_a_silent_tool(bench, tmp_path, monkeypatch):
  monkeypatch.setenv('PATH', _fake_smi(tmp_path, 'sleep 30\n') + os.pathsep + os.environ['PATH'])
  s = bench.ClockSampler(0)
  s.wait_first_sample(timeout=0.3)
  out = s.stop()
  assert out['sm_mhz'] is None and out['reasons'] == ['no samples']


def test_clock_sampler_ignores_other_gpus_and_reports_slowdown(bench, tmp_path, monkeypatch):
  body = ('echo "1, 1200, 1965, 300.0, 0x8, Active, Not Active, Not Active, Not Active"\n'
          'echo "0, 1500, 1965, 300.0, 0x8, Active, Not Active, Not Active, Not Active"\n'
          'sleep 30\n')
  monkeypatch.setenv('PATH', _fake_smi(tmp_path, body) + os.pathsep + os.environ['PATH'])
  s = bench.ClockSampler(0)
  s.wait_first_sample(timeout=2.0)
  time.sleep(0.1)
  out = s.stop()
  assert out['sm_mhz'] == 1500.0 and out['reasons'] == ['hw_slowdown'] and out['samples'] == 1


def test_physical_gpu_index_follows_cuda_visible_devices(bench, monkeypatch):
  monkeypatch.delenv('CUDA_VISIBLE_DEVICES', raising=False)
  assert bench.physical_gpu_index(2) == 2
  monkeypatch.setenv('CUDA_VISIBLE_DEVICES', '5,7')
  assert bench.physical_gpu_index(0) == 5 and bench.physical_gpu_index(1) == 7
  assert bench.physical_gpu_index(3) == 3            # beyond the list: the local index itself
  monkeypatch.setenv('CUDA_VISIBLE_DEVICES', 'GPU-8f2c,GPU-11aa')
  assert bench.physical_gpu_index(1) == 1            # UUIDs: nothing to translate


def test_conv_work_counts_the_reference_dense_flops(bench):
  # octree/octree/octree_conv.cpp:287-289: a GEMM of [Cout, Cin*K] x [Cin*K, H]
  flops, byts = bench.conv_work({'ks': [3, 3, 3], 'cin': 8, 'cout': 32}, 1000)
  assert flops == 2.0 * 32 * 8 * 27 * 1000
  assert byts == (8 + 32) * 1000 * 2 + 32 * 1000 + 32 * 8 * 27 * 2
  flops, byts = bench.conv_work({'ks': [1, 1, 1], 'cin': 16, 'cout': 64}, 10)
  assert flops == 2.0 * 64 * 16 * 10 and byts == (16 + 64) * 10 * 2 + 64 * 16 * 2
