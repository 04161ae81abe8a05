"""Medilix on the GPU with the engine's kernels, in float32 and bfloat16, against
tests/plain_medilix.py: each mechanism alone, then whole models under every kind of schedule."""

import pytest
import torch

import medilix_cases as mc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_alone(ops, dtype):
    mc.case_mixer_alone(dtype, ops, DEV, "mlstm")
    mc.case_mixer_alone(dtype, ops, DEV, "mlstm", heads=1, dim=40, vdim=8, gate_cap=2.0)
    mc.case_mixer_alone(dtype, ops, DEV, "mlstm", heads=2, dim=128, vdim=72, gate_cap=15.0, T=80, cuts=(33, 1, 2, 44))
    mc.case_mixer_alone(dtype, ops, DEV, "wkv")
    mc.case_mixer_alone(dtype, ops, DEV, "wkv", heads=1, dim=40, rank=3)
    mc.case_mixer_alone(dtype, ops, DEV, "wkv", heads=2, dim=64, rank=16, T=80, cuts=(33, 1, 2, 44))
    mc.case_mixer_alone(dtype, ops, DEV, "attention")
    mc.case_mixer_alone(dtype, ops, DEV, "attention", page_size=4, heads=2, kv_heads=2, dim=16, vdim=8, mask=None)
    mc.case_mixer_alone(dtype, ops, DEV, "attention", heads=4, kv_heads=1, dim=8, vdim=24,
                        mask=dict(size=5, keep_first=11))
    mc.case_mixer_alone(dtype, ops, DEV, "attention", page_size=16, T=150, cuts=(70, 1, 2, 77), heads=8, kv_heads=2,
                        dim=64, vdim=64, scale=0.125, mask=dict(size=40, keep_first=16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_memories(ops, dtype):
    mc.case_stabilised_memory(dtype, ops, DEV)
    mc.case_stabilised_memory(dtype, ops, DEV, H=2, D=128, Dv=40, cap=12.0)
    mc.case_stabilised_memory(dtype, ops, DEV, H=1, D=7, Dv=33, cap=3.0)
    mc.case_bonus_memory(dtype, ops, DEV)
    mc.case_bonus_memory(dtype, ops, DEV, H=2, D=64, Dv=64)
    mc.case_bonus_memory(dtype, ops, DEV, H=1, D=7, Dv=33)
    mc.case_memories_remember_a_far_token(dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_edges(ops, dtype):
    mc.case_attention_edges(dtype, ops, DEV)
    mc.case_attention_edges(dtype, ops, DEV, window=8, keep=1, page_size=8, heads=1, kv_heads=1, D=20, Dv=8)
    mc.case_attention_edges(dtype, ops, DEV, window=16, keep=5, page_size=16, heads=6, kv_heads=2, D=48, Dv=96, T=70)
    mc.case_attention_edges(dtype, ops, DEV, window=33, keep=16, page_size=16, heads=8, kv_heads=2, D=64, Dv=64, T=120)
    # keys and values of one size, dense rows: in bfloat16 the split-KV and the tensor-core prompt kernels
    mc.case_attention_edges(dtype, ops, DEV, window=33, keep=16, page_size=16, heads=8, kv_heads=2, D=64, Dv=64, T=120,
                            dense_out=True)
    mc.case_attention_edges(dtype, ops, DEV, window=150, keep=70, page_size=16, heads=4, kv_heads=1, D=128, Dv=128,
                            T=330, dense_out=True, decode_slices=3)
    mc.case_attention_edges(dtype, ops, DEV, window=70, keep=130, page_size=32, heads=2, kv_heads=2, D=64, Dv=64,
                            T=300, dense_out=True, decode_slices=2)
    mc.case_attention_edges(dtype, ops, DEV, window=70, keep=9, page_size=16, heads=2, kv_heads=1, D=256, Dv=256,
                            T=160, dense_out=True, decode_slices=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_state_and_norm(ops, dtype):
    mc.case_token_state(dtype, ops, DEV)
    mc.case_token_state(dtype, ops, DEV, buckets=1, mul_prev=0, mul_cur=1)
    mc.case_token_state(dtype, ops, DEV, W=200, vocab=300, buckets=1009, mul_prev=37, mul_cur=11)
    mc.case_token_state(dtype, ops, DEV, W=36)  # rows that are no multiple of 8 values: one value a thread
    mc.case_grouped_norm(dtype, ops, DEV)
    mc.case_grouped_norm(dtype, ops, DEV, W=240)  # groups of a multiple of 8 values: eight values a thread
    mc.case_grouped_norm(dtype, ops, DEV, W=4080)


@pytest.mark.parametrize("dtype", DTYPES)
def test_routing_and_feed_forwards(ops, dtype):
    mc.case_routing(dtype, ops, DEV)
    mc.case_feed_forwards_alone(dtype, ops, DEV)
    mc.case_feed_forwards_alone(dtype, ops, DEV, T=300)
    mc.case_feed_forwards_alone(dtype, ops, DEV, experts=3, identity=0, top=1, groups=None)
    mc.case_feed_forwards_alone(dtype, ops, DEV, experts=2, identity=4, top=6, groups=(3, 3))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_schedules(tmp_path, ops, name, dtype):
    mc.case_schedules(tmp_path, name, dtype, ops, DEV)


@pytest.mark.parametrize("name", ["A", "C"])
def test_residual_after_every_run(tmp_path, ops, name):
    mc.case_residual_after_every_run(tmp_path, name, ops, DEV)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_schedules_through_captured_decode_steps(tmp_path, ops, name):
    mc.case_schedules(tmp_path, name, "bfloat16", ops, DEV, cuda_graph=True)
    mc.case_schedules(tmp_path, name, "float32", ops, DEV, cuda_graph=True, lengths=(40, 5, 33))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decode(tmp_path, ops, dtype):
    mc.case_long_decode(tmp_path, "A", dtype, ops, DEV, total=200, cuda_graph=True)
    mc.case_long_decode(tmp_path, "B", dtype, ops, DEV, total=120)
    mc.case_long_decode(tmp_path, "D", dtype, ops, DEV, total=120, cuda_graph=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(tmp_path, ops, dtype):
    mc.case_first_tokens(tmp_path, "A", dtype, ops, DEV)
    mc.case_first_tokens(tmp_path, "B", dtype, ops, DEV)
    mc.case_first_tokens(tmp_path, "C", dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuda_graph", [False, True])
def test_greedy_generation_under_the_scheduler(tmp_path, ops, dtype, cuda_graph):
    mc.case_greedy_generation(tmp_path, "A", dtype, ops, DEV, cuda_graph=cuda_graph)
    mc.case_greedy_generation(tmp_path, "C", dtype, ops, DEV, cuda_graph=cuda_graph)


def test_trace_replay_program_on_a_medilix_folder(tmp_path, ops):
    """bin/trace_run as a subprocess: the model class is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    folder = mc.make_dir(tmp_path, "C")
    toks = mc.requests_for("C", (20,))["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:13], "want": [0, 12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[13:], "want": [6]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "64"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want, tol = mc.expected(folder, {"a": toks}, "float32")
    V = mc.CONFIGS["C"]["config"].vocab
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    assert float((got0 - want["a"][[0, 12]]).abs().max()) <= tol
    assert float((got1 - want["a"][[19]]).abs().max()) <= tol


def test_command_line_on_a_medilix_folder(tmp_path):
    """``python -m qwen3_runtime_b200.cli`` generates greedily from a Medilix folder what the plain model does."""
    import os
    import subprocess
    import sys

    import plain_medilix as pl

    folder = mc.make_dir(tmp_path, "A")
    raw, t = mc.read_dir(folder)
    prompt = [5, 6, 7, 8, 9]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "qwen3_runtime_b200.cli", "--model", str(folder), "--max-tokens", "6", "--dtype",
           "float32", "--prompt-tokens", *map(str, prompt), "--num-kv-blocks", "16", "--no-cuda-graph"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = dict(line.split(" ", 1) for line in proc.stdout.strip().splitlines())
    got = [int(x) for x in lines["runtime"].strip("[]").split(",")]
    assert len(got) == 6
    seq = list(prompt)
    for tok in got:  # every token is the plain model's best (or within float32 rounding of it) given the tokens before
        row = pl.forward(raw, t, seq)[-1]
        assert float(row.max() - row[tok]) <= 1e-4 * max(1.0, float(row.abs().max()))
        seq.append(tok)
