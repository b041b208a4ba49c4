"""The Engine adapter (adapter/engine_b200.cpp: rapidllm::cuda_gen::Engine over the rl_* C ABI) compiles
against the reference's own headers and links against the library with no symbol left open.  Needs
the reference tree (its headers and src/ir/model_desc.cpp are compiled where they lie); skipped when
it is not there.  No GPU is touched."""
import os
import shutil
import subprocess

import pytest

from conftest import ROOT


def _reference():
    import oracle
    return oracle.reference_tree()


def test_adapter_compiles_and_links_against_the_reference_headers(tmp_path):
    ref = _reference()
    if not ref:
        pytest.skip("reference tree not present")
    gxx = shutil.which("g++")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    if not gxx or not os.path.exists(os.path.join(cuda, "include", "cuda_runtime_api.h")):
        pytest.skip("g++ or the CUDA headers are missing")
    from rapidllm_b200 import _lib
    _lib.lib()                                                    # the library must exist to link against
    inc = ["-I" + os.path.join(ref, "include"), "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include")]
    obj = str(tmp_path / "engine_b200.o")
    subprocess.run([gxx, "-std=c++20", "-Wall", "-Werror", "-fPIC"] + inc +
                   ["-c", os.path.join(ROOT, "adapter", "engine_b200.cpp"), "-o", obj], check=True)
    md = str(tmp_path / "model_desc.o")
    subprocess.run([gxx, "-std=c++20", "-fPIC", inc[0], "-c", os.path.join(ref, "src", "ir", "model_desc.cpp"), "-o", md],
                   check=True)
    # every symbol resolved: the Engine interface, ModelDesc::mixer_slot, the rl_* ABI and the CUDA runtime
    subprocess.run([gxx, "-shared", "-o", str(tmp_path / "libengine_b200.so"), obj, md,
                    "-L" + os.path.dirname(_lib.LIB_PATH), "-lrl_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart",
                    "-Wl,-z,defs"], check=True)
    # the two symbols a RapidLLM build takes from this file instead of cuda_engine.cu / the stub
    syms = subprocess.run(["nm", "-C", "--defined-only", obj], check=True, capture_output=True, text=True).stdout
    assert "rapidllm::cuda_gen::available()" in syms
    assert "rapidllm::cuda_gen::Engine::create(" in syms
