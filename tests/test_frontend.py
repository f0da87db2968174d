"""The C++ front end (include/fused_kernel/): it compiles with g++ -std=c++20, rejects ill-typed chains at compile time
like the reference does, and — on a GPU — reproduces the oracle bit for bit on the benchmark pipelines written with the
reference's own API spellings (tests/cpp/frontend_test.cpp)."""
import os
import subprocess
import tempfile

import pytest

from conftest import ROOT

CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
HEAD = '''
#include <fused_kernel/algorithms/basic_ops/arithmetic.h>
#include <fused_kernel/algorithms/basic_ops/cast.h>
#include <fused_kernel/algorithms/basic_ops/memory_operations.h>
#include <fused_kernel/algorithms/image_processing/crop.h>
#include <fused_kernel/algorithms/image_processing/resize.h>
#include <fused_kernel/algorithms/image_processing/saturate.h>
#include <fused_kernel/fused_kernel.h>
using namespace fk;
'''


def syntax_check(body: str):
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp")
        open(src, "w").write(HEAD + "void f(Stream& stream, Ptr2D<uchar3>& in, Tensor<uchar3>& out8, Tensor<float3>& out32) {\n" + body + "\n}\n")
        return subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"), src],
                              capture_output=True, text=True)


def test_frontend_program_builds():
    import frontend_build
    assert os.path.exists(frontend_build.build())


def test_well_typed_chain_compiles():
    r = syntax_check("executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Crop<>::build(Rect(0,0,8,8)),"
                     " Resize<InterpolationType::INTER_LINEAR>::build(Size(4,4)), Mul<float3>::build(make_set<float3>(2.f)), TensorWrite<float3>::build(out32));")
    assert r.returncode == 0, r.stderr


@pytest.mark.parametrize("body,needle", [
    # Mul<float3> straight after a uchar3 read: InputType != OutputType of the previous operation
    ("executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Mul<float3>::build(make_set<float3>(2.f)), TensorWrite<float3>::build(out32));",
     "InputType is not the OutputType"),
    # float3 result written through a uchar3 write
    ("executeOperations<TransformDPP<>>(stream, PerThreadRead<ND::_2D, uchar3>::build(in), Cast<uchar3, float3>::build(), TensorWrite<uchar3>::build(out8));",
     "Write's InputType"),
    # a chain that does not start with a Read
    ("executeOperations<TransformDPP<>>(stream, Cast<uchar3, float3>::build(), TensorWrite<float3>::build(out32));", "first IOp must be a complete Read"),
    # the CPU back end is not provided by this library
    ("Stream_<ParArch::CPU> s; executeOperations<TransformDPP<ParArch::CPU>>(s, PerThreadRead<ND::_2D, uchar3>::build(in), TensorWrite<uchar3>::build(out8));",
     "GPU_NVIDIA only"),
])
def test_ill_typed_chains_are_compile_errors(body, needle):
    r = syntax_check(body)
    assert r.returncode != 0 and needle in r.stderr, r.stderr[-2000:]


@pytest.mark.gpu
def test_frontend_pipelines_match_oracle_on_gpu():
    import frontend_build
    exe = frontend_build.build()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout + r.stderr
