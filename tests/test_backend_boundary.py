"""Runs the C++ boundary test: the W4A32 op behind the reference's own plugin API
(MllmEngineCtx, BackendBase, nn::Module / nn::Linear, ParameterLoader, ir::PassManager), built by
mllm-advanced_b200/backend/Makefile against the reference's real classes.  The binary is built where
the reference tree exists and travels as a prebuilt file; its source is tests/backend/boundary_test.cpp."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "backend_boundary_test")


@pytest.mark.skipif(not os.path.exists(BIN), reason="oracle/_ref/backend_boundary_test not built (needs the reference tree)")
def test_quantization_pass_through_reference_pass_manager_host_only():
    """CudaQuantizationPass run by the reference's ir::PassManager on flat IR modules (Linear, the W4A16 sibling,
    Conv3D): the blob's nibble and scale sections equal the oracle's quantizer bit for bit; and the quantizer
    tool's whole flow (tools::createFlatModule + the pass + the reference's CommonParamQuantizePass + mllm::write)
    over a generated 28-layer parameter file, read back with mllm::load.  No GPU involved."""
    r = subprocess.run([BIN, "--host-only"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "BOUNDARY TEST PASSED" in r.stdout and r.stdout.count("[ ok ]") >= 60
    assert "createFlatModule found 196 linears, the pass quantized 196" in r.stdout
    assert "196 linear blobs bit-identical to the oracle's quantizer" in r.stdout


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(BIN), reason="oracle/_ref/backend_boundary_test not built (needs the reference tree)")
def test_linear_op_through_reference_plugin_api():
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(r.stdout[-4000:])
    print(r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "BOUNDARY TEST PASSED" in r.stdout
    assert "FAIL" not in r.stdout.replace("0 failures", "")
    assert r.stdout.count("nn::Conv3D forward") == 3  # the Conv3D op ran through nn::Conv3D on the CUDA backend
