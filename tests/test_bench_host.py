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
