"""Build libocnn_b200.so (CUDA kernels + C ABI, sm_100a only) and the `ocnn.nn` torch extension
in-tree.  Usage:  python o-cnn_b200/build.py [--lib-only] [--force]"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OBJ = os.path.join(HERE, 'build', 'obj')
LIB = os.path.join(HERE, 'libocnn_b200.so')

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '--expt-relaxed-constexpr']
# files whose floating-point results must round exactly like the reference's scalar CPU code
NO_FMA = {'build.cu', 'points.cu'}


def _newer(target, deps):
  if not os.path.exists(target):
    return True
  t = os.path.getmtime(target)
  return any(os.path.getmtime(d) > t for d in deps)


def _headers():
  hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.h', '.cuh'))]
  hs.append(os.path.join(HERE, '..', 'include', 'ocnn_b200.h'))
  return hs


def _compile(src, force, verbose):
  obj = os.path.join(OBJ, os.path.basename(src) + '.o')
  if not force and not _newer(obj, [src] + _headers()):
    return obj, ''
  cmd = ['nvcc'] + NVCC_FLAGS + (['--fmad=false'] if os.path.basename(src) in NO_FMA else [])
  if verbose:
    cmd += ['-Xptxas', '-v']
  cmd += ['-c', src, '-o', obj]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError('nvcc failed for %s:\n%s\n%s' % (src, res.stdout, res.stderr))
  return obj, res.stderr


def build_lib(force=False, verbose=False):
  os.makedirs(OBJ, exist_ok=True)
  srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith('.cu'))
  with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
    results = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
  objs = [o for o, _ in results]
  if verbose:
    for _, log in results:
      sys.stderr.write(log)
  if force or _newer(LIB, objs):
    cmd = ['nvcc', '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', LIB] + objs
    subprocess.check_call(cmd)
  return LIB


def build_ext(force=False):
  """The torch extension `ocnn.nn` (pybind11, host C++ only) linked against libocnn_b200.so."""
  import sysconfig
  import torch
  from torch.utils import cpp_extension
  src = os.path.join(HERE, 'torch_ext', 'ocnn_nn.cpp')
  suffix = sysconfig.get_config_var('EXT_SUFFIX')
  out = os.path.join(HERE, 'ocnn', 'nn' + suffix)
  deps = [src, os.path.join(HERE, '..', 'include', 'ocnn_b200.h'), LIB]
  if not force and not _newer(out, deps):
    return out
  inc = ['-I' + p for p in cpp_extension.include_paths()]
  inc += ['-I' + sysconfig.get_paths()['include'], '-I' + os.path.join(HERE, '..', 'include')]
  tlib = os.path.join(os.path.dirname(torch.__file__), 'lib')
  cuda_inc = '/usr/local/cuda/include'
  cmd = ['g++', '-O2', '-std=c++17', '-fPIC', '-shared', '-DTORCH_EXTENSION_NAME=nn',
         '-DTORCH_API_INCLUDE_EXTENSION_H', '-D_GLIBCXX_USE_CXX11_ABI=%d' % int(torch._C._GLIBCXX_USE_CXX11_ABI),
         '-I' + cuda_inc] + inc + [src, '-o', out, '-L' + HERE, '-locnn_b200',
         '-L' + tlib, '-ltorch', '-ltorch_cpu', '-ltorch_python', '-lc10', '-lc10_cuda', '-ltorch_cuda',
         '-Wl,-rpath,$ORIGIN/..', '-Wl,-rpath,' + tlib]
  subprocess.check_call(cmd)
  return out


if __name__ == '__main__':
  force = '--force' in sys.argv
  build_lib(force=force, verbose='--verbose' in sys.argv)
  if '--lib-only' not in sys.argv:
    build_ext(force=force)
  print('built', LIB)
