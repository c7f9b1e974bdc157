"""The C++ host side: op registry, ONNX subset reader and the op_test_runner-compatible harness.

CPU part: the harness parses a model and a manifest (`--parse-only`), rejects malformed ones.
GPU part: the harness runs MatMulQ4K end to end from files and the result is checked against
the CPU checker -- the way a script written against the reference's op_test_runner would use it.
"""
import json
import os
import subprocess

import numpy as np
import pytest

import onnx_writer as ow
from backpack_b200 import synth
from oracle import q4k_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "backpack_b200", "bin", "bpq4k_op_test_runner")


def write_case(tmp, N, K, x, raw, bias, w_as_initializer, op="MatMulQ4K", block_bytes=144):
    tmp.mkdir(parents=True, exist_ok=True)
    indir, outdir = tmp / "in", tmp / "out"
    indir.mkdir()
    model = ow.matmul_q4k_model(N, K, x.shape, raw if w_as_initializer else None, bias is not None, op, block_bytes)
    (tmp / "m.onnx").write_bytes(model)
    inputs = [{"name": "X", "dtype": "float32", "shape": list(x.shape)}]
    x.tofile(indir / "X.bin")
    if not w_as_initializer:
        inputs.append({"name": "W", "dtype": "uint8", "shape": list(raw.shape)})
        raw.tofile(indir / "W.bin")
    if bias is not None:
        inputs.append({"name": "Bias", "dtype": "float32", "shape": [N]})
        bias.tofile(indir / "Bias.bin")
    (indir / "manifest.json").write_text(json.dumps({"inputs": inputs}))
    return str(tmp / "m.onnx"), str(indir), str(outdir)


def test_runner_exists_and_usage():
    assert os.path.isfile(RUNNER), "build it with `make -C backpack_b200/host`"
    r = subprocess.run([RUNNER], capture_output=True, text=True)
    assert r.returncode == 1 and "Usage:" in r.stderr and "<model.onnx> <input_dir> <output_dir>" in r.stderr


def test_parse_only_reads_model_and_manifest(tmp_path):
    N, K = 12, 512
    raw = synth.make_q4k_weights(N, K, 1)
    x = synth.make_activations(3, K, 2)
    bias = np.arange(N, dtype=np.float32)
    model, indir, outdir = write_case(tmp_path / "a", N, K, x, raw, bias, w_as_initializer=True)
    r = subprocess.run([RUNNER, "--parse-only", model, indir, outdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert "op=MatMulQ4K registered=1 inputs=3 outputs=1" in out
    assert "K=512" in out and "N=12" in out
    assert f"initializer W dtype=uint8 bytes={raw.size}" in out
    assert "graph-input X dtype=float32 rank=2" in out and "graph-input Bias" in out
    assert "graph-input W" not in out          # an initializer is a weight, not a runtime input
    assert "graph-output Y dtype=float32 rank=2" in out
    assert "manifest-input X dtype=float32 rank=2" in out
    assert out.strip().endswith("OK")


def test_parse_only_knows_the_sibling_ops(tmp_path):
    for op, qtype in (("MatMulQ5K", orc.Q5_K), ("MatMulQ6K", orc.Q6_K)):
        N, K = 6, 512
        raw = synth.make_kq_weights(qtype, N, K, 1).reshape(N, -1)
        x = synth.make_activations(2, K, 2)
        model, indir, outdir = write_case(tmp_path / op, N, K, x, raw, None, True, op, synth.KQ_BLOCK_BYTES[qtype])
        r = subprocess.run([RUNNER, "--parse-only", model, indir, outdir], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        assert f"op={op} registered=1 inputs=2 outputs=1" in r.stdout
        assert f"initializer W dtype=uint8 bytes={raw.size}" in r.stdout


def test_parse_only_rejects_garbage(tmp_path):
    (tmp_path / "in").mkdir()
    (tmp_path / "in" / "manifest.json").write_text('{"inputs": []}')
    (tmp_path / "bad.onnx").write_bytes(b"\xff\xff\xff\xff\xff\xff\xff\xff\xff\xff\xff\xff")
    r = subprocess.run([RUNNER, "--parse-only", str(tmp_path / "bad.onnx"), str(tmp_path / "in"), str(tmp_path / "o")],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "Failed to load" in r.stderr
    r = subprocess.run([RUNNER, "--parse-only", str(tmp_path / "missing.onnx"), str(tmp_path / "in"), str(tmp_path / "o")],
                       capture_output=True, text=True)
    assert r.returncode == 1
    good = ow.matmul_q4k_model(4, 256, (1, 256), None, False)
    (tmp_path / "g.onnx").write_bytes(good)
    (tmp_path / "in" / "manifest.json").write_text("{not json")
    r = subprocess.run([RUNNER, "--parse-only", str(tmp_path / "g.onnx"), str(tmp_path / "in"), str(tmp_path / "o")],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "Cannot parse" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("w_as_initializer", [True, False])
@pytest.mark.parametrize("M,N,K,with_bias", [(1, 40, 1024, False), (5, 9, 512, True), (1, 4096, 4096, False)])
def test_runner_end_to_end(tmp_path, M, N, K, with_bias, w_as_initializer):
    raw = synth.make_q4k_weights(N, K, 7)
    x = synth.make_activations(M, K, 8)
    bias = (np.arange(N) * 0.01).astype(np.float32) if with_bias else None
    model, indir, outdir = write_case(tmp_path / "c", N, K, x, raw, bias, w_as_initializer)
    r = subprocess.run([RUNNER, model, indir, outdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == "OK" and "Execute:" in r.stderr
    man = json.loads(open(os.path.join(outdir, "manifest.json")).read())
    assert man == {"outputs": [{"name": "Y", "dtype": "float32", "shape": [M, N]}]}
    y = np.fromfile(os.path.join(outdir, "Y.bin"), np.float32).reshape(M, N)
    want = orc.matmul(x, raw, bias, N, K, threads=4)
    assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 1e-3
    assert np.abs(y - want).max() <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("op,qtype", [("MatMulQ5K", orc.Q5_K), ("MatMulQ6K", orc.Q6_K)])
@pytest.mark.parametrize("M,N,K,with_bias,w_as_initializer",
                         [(1, 40, 1024, False, True), (5, 9, 512, True, False), (3, 1024, 4096, False, True),
                          (40, 256, 2048, True, True)])
def test_runner_sibling_ops_end_to_end(tmp_path, op, qtype, M, N, K, with_bias, w_as_initializer):
    """MatMulQ5K / MatMulQ6K take W in the file format of their type (Q6_K: 210-byte blocks, re-spaced on the device)."""
    raw = synth.make_kq_weights(qtype, N, K, 17).reshape(N, -1)
    x = synth.make_activations(M, K, 18)
    bias = (np.arange(N) * 0.01).astype(np.float32) if with_bias else None
    model, indir, outdir = write_case(tmp_path / "c", N, K, x, raw, bias, w_as_initializer, op, synth.KQ_BLOCK_BYTES[qtype])
    r = subprocess.run([RUNNER, model, indir, outdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == "OK"
    man = json.loads(open(os.path.join(outdir, "manifest.json")).read())
    assert man == {"outputs": [{"name": "Y", "dtype": "float32", "shape": [M, N]}]}
    y = np.fromfile(os.path.join(outdir, "Y.bin"), np.float32).reshape(M, N)
    want = orc.kq_matmul(qtype, x, raw.reshape(-1), bias, N, K, threads=4)
    assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 1e-3
    assert np.abs(y - want).max() <= 2e-2


@pytest.mark.gpu
def test_runner_missing_input_means_zeros_and_bad_shape_leaves_output_invalid(tmp_path):
    N, K = 8, 256
    raw = synth.make_q4k_weights(N, K, 1)
    x = synth.make_activations(1, K, 2)
    model, indir, outdir = write_case(tmp_path / "z", N, K, x, raw, None, w_as_initializer=True)
    os.remove(os.path.join(indir, "X.bin"))                # missing file -> zero tensor
    r = subprocess.run([RUNNER, model, indir, outdir], capture_output=True, text=True)
    assert r.returncode == 0 and "Cannot open input" in r.stderr
    assert (np.fromfile(os.path.join(outdir, "Y.bin"), np.float32) == 0).all()
    # K attribute that does not match X: the op returns early, the harness reports the output invalid
    bad = ow.matmul_q4k_model(N, 512, (1, 256), raw, False)
    open(model, "wb").write(bad)
    x.tofile(os.path.join(indir, "X.bin"))
    r = subprocess.run([RUNNER, model, indir, str(tmp_path / "o2")], capture_output=True, text=True)
    assert r.returncode == 0 and "Output 'Y' not valid" in r.stderr
    assert json.loads(open(tmp_path / "o2" / "manifest.json").read()) == {"outputs": []}
