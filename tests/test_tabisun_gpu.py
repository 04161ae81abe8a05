"""Tabisun on the GPU with the engine's kernels, in float32 and bfloat16, against tests/plain_tabisun.py:
each mechanism alone, then whole models under every kind of schedule."""

import pytest
import torch

import tabisun_cases as tc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_alone(ops, dtype):
    tc.case_mixer_alone(dtype, ops, DEV, "attention")
    tc.case_mixer_alone(dtype, ops, DEV, "attention", page_size=4, heads=2, kv_heads=2, dim=16, vdim=16, chunk=None)
    tc.case_mixer_alone(dtype, ops, DEV, "attention", heads=3, kv_heads=1, dim=8, vdim=40, chunk=7, diff=0.9)
    tc.case_mixer_alone(dtype, ops, DEV, "attention", page_size=16, T=150, cuts=(70, 1, 2, 77), heads=4, kv_heads=1,
                        dim=64, vdim=128, scale=0.125, chunk=48)
    tc.case_mixer_alone(dtype, ops, DEV, "attention_2")
    tc.case_mixer_alone(dtype, ops, DEV, "attention_2", page_size=4, heads=2, kv_heads=2, dim=20, softcap=None,
                        rot=None)
    tc.case_mixer_alone(dtype, ops, DEV, "attention_2", page_size=16, T=150, cuts=(70, 1, 2, 77), heads=8, kv_heads=2,
                        dim=64, scale=0.125, softcap=30.0,
                        rot=tc.RotaryConfig(dims=32, base=5e5, scaling=tc._wave(8.0, 1.0, 4.0, 256.0)))
    tc.case_mixer_alone(dtype, ops, DEV, "attention_2", page_size=16, T=150, cuts=(70, 1, 2, 77), heads=4, kv_heads=1,
                        dim=128, scale=0.09, softcap=50.0,
                        rot=tc.RotaryConfig(dims=128, base=1e4, scaling=tc._wave(8.0, 1.0, 4.0, 64.0)))
    tc.case_mixer_alone(dtype, ops, DEV, "latent_attention")
    tc.case_mixer_alone(dtype, ops, DEV, "latent_attention", heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=16,
                        rot=tc.RotaryConfig(dims=4, base=100.0))
    tc.case_mixer_alone(dtype, ops, DEV, "latent_attention", page_size=16, T=150, cuts=(70, 1, 2, 77), heads=4, dim=32,
                        rot_dim=16, vdim=32, kv_rank=64, scale=0.15,
                        rot=tc.RotaryConfig(dims=16, base=1e4, scaling=tc._ramp(4.0, 128.0, 32.0, 1.0)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_edges(ops, dtype):
    tc.case_differential_edges(dtype, ops, DEV)
    tc.case_differential_edges(dtype, ops, DEV, chunk=8, page_size=8, heads=1, kv_heads=1, D=20, Dv=8)
    tc.case_differential_edges(dtype, ops, DEV, chunk=33, page_size=16, heads=6, kv_heads=2, D=48, Dv=96, T=130)
    # sizes that in bfloat16 run the tensor-core prompt kernel and the sliced decode kernel (groups of 4, 8, 2, 1;
    # several slices; chunks that are no multiple of the key tile; no chunk at all)
    tc.case_differential_edges(dtype, ops, DEV, chunk=64, page_size=16, heads=4, kv_heads=1, D=64, Dv=128, T=200)
    tc.case_differential_edges(dtype, ops, DEV, chunk=200, page_size=16, heads=8, kv_heads=1, D=32, Dv=64, T=700)
    tc.case_differential_edges(dtype, ops, DEV, chunk=100, page_size=8, heads=4, kv_heads=2, D=64, Dv=64, T=330)
    tc.case_differential_edges(dtype, ops, DEV, chunk=129, page_size=32, heads=2, kv_heads=2, D=128, Dv=128, T=420)
    tc.case_differential_edges(dtype, ops, DEV, chunk=70, page_size=16, heads=4, kv_heads=2, D=32, Dv=128, T=230)
    tc.case_differential_edges(dtype, ops, DEV, chunk=70, page_size=16, heads=2, kv_heads=1, D=128, Dv=64, T=230)
    # sizes that those kernels refuse although their groups and alignments fit: the general kernel serves them
    tc.case_differential_edges(dtype, ops, DEV, chunk=40, page_size=16, heads=4, kv_heads=1, D=16, Dv=96, T=130)
    tc.case_differential_edges(dtype, ops, DEV, chunk=40, page_size=16, heads=2, kv_heads=1, D=64, Dv=256, T=130)
    tc.case_capped_far_key(dtype, ops, DEV)
    tc.case_capped_far_key(dtype, ops, DEV, chunk=100)
    tc.case_capped_far_key(dtype, ops, DEV, heads=8, kv_heads=2, D=64, T=400)
    tc.case_capped_far_key(dtype, ops, DEV, heads=4, kv_heads=1, D=128, T=400, softcap=5.0)
    tc.case_latent_far_key_and_sink(dtype, ops, DEV)
    tc.case_latent_far_key_and_sink(dtype, ops, DEV, page_size=8, heads=3, rank=44, rot=12, T=200)  # the general kernel


@pytest.mark.parametrize("dtype", DTYPES)
def test_norms_and_rotations(ops, dtype):
    tc.case_layer_norms(dtype, ops, DEV)
    tc.case_rotations(dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_schedules(tmp_path, ops, name, dtype):
    tc.case_schedules(tmp_path, name, dtype, ops, DEV)


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_residual_after_every_run(tmp_path, ops, name):
    tc.case_residual_after_every_run(tmp_path, name, ops, DEV)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_schedules_through_captured_decode_steps(tmp_path, ops, name):
    tc.case_schedules(tmp_path, name, "bfloat16", ops, DEV, cuda_graph=True)
    tc.case_schedules(tmp_path, name, "float32", ops, DEV, cuda_graph=True, lengths=(40, 5, 33))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decode(tmp_path, ops, dtype):
    tc.case_long_decode(tmp_path, "A", dtype, ops, DEV, total=200, cuda_graph=True)
    tc.case_long_decode(tmp_path, "B", dtype, ops, DEV, total=120)
    tc.case_long_decode(tmp_path, "D", dtype, ops, DEV, total=330, cuda_graph=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(tmp_path, ops, dtype):
    tc.case_first_tokens(tmp_path, "A", dtype, ops, DEV)
    tc.case_first_tokens(tmp_path, "B", dtype, ops, DEV)
    tc.case_first_tokens(tmp_path, "C", dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuda_graph", [False, True])
def test_greedy_generation_under_the_scheduler(tmp_path, ops, dtype, cuda_graph):
    tc.case_greedy_generation(tmp_path, "A", dtype, ops, DEV, cuda_graph=cuda_graph)
    tc.case_greedy_generation(tmp_path, "D", dtype, ops, DEV, cuda_graph=cuda_graph)


def test_bfloat16_steps_take_the_specialised_kernels(tmp_path, ops):
    """With sizes they take, a bfloat16 model runs prompt portions on the tensor-core kernels and decode steps on
    the sliced differential kernel, the split-KV kernel in the form that also norms, turns and stores the newest
    token (its values read where its keys are) and the tensor-core kernel over latent rows."""
    from helpers import run_trace, trace_tail_decode

    folder = tc.make_dir(tmp_path, "D")
    launched, new_tokens = [], []
    call, decode = ops._call, ops.paged_attention_decode

    def call_spy(group, name, what, *args):
        launched.append(what)
        return call(group, name, what, *args)

    def decode_spy(*args, **kw):
        new_tokens.append(kw.get("new_token"))
        return decode(*args, **kw)

    ops._call, ops.paged_attention_decode = call_spy, decode_spy
    try:
        rt = tc.runtime(folder, "D", "bfloat16", ops, DEV, pages=16)
        run_trace(rt, trace_tail_decode(tc.requests_for("D", (70,)), tail=5))
    finally:
        del ops._call, ops.paged_attention_decode
    for kernel in ("differential_attention_tc", "differential_attention_decode", "paged_attention_prefill",
                   "paged_attention_decode_fused", "latent_attention_tc"):
        assert kernel in launched, f"{kernel} was not launched: {sorted(set(launched))}"
    assert "differential_attention" not in launched and "paged_attention" not in launched  # the general kernels
    assert new_tokens and all(nt is not None and nt["values_are_keys"] and nt["cos"] is not None for nt in new_tokens)


def test_trace_replay_program_on_a_tabisun_folder(tmp_path, ops):
    """bin/trace_run as a subprocess: the model class is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    folder = tc.make_dir(tmp_path, "C")
    toks = tc.requests_for("C", (40,))["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:31], "want": [0, 30]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[31:], "want": [8]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "64"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want, tol = tc.expected(folder, {"a": toks}, "float32")
    V = tc.CONFIGS["C"]["config"].vocab
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    assert float((got0 - want["a"][[0, 30]]).abs().max()) <= tol
    assert float((got1 - want["a"][[39]]).abs().max()) <= tol


def test_command_line_on_a_tabisun_folder(tmp_path):
    """``python -m qwen3_runtime_b200.cli`` generates greedily from a Tabisun folder what the plain model does."""
    import os
    import subprocess
    import sys

    import plain_tabisun as pl

    folder = tc.make_dir(tmp_path, "A")
    raw, t = tc.read_dir(folder)
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
        row = pl.forward(raw, t, seq)[-1].float()
        assert float(row.max() - row[tok]) <= 1e-4 * max(1.0, float(row.abs().max()))
        seq.append(tok)
