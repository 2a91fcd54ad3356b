"""The C++ drop-in: the reference's own programs, compiled unchanged against this repository's CudaEngine
headers (neuralnet.cpp_b200/engine/), run on the GPU with --cuda.

The binaries are built from the reference sources by `make -C oracle` into oracle/_ref/engine/ (test
infrastructure; they carry the reference CPU engine too, which is what each program checks against):
  engine_check            every ComputeEngine virtual, reference CpuEngine vs CudaEngine on the same inputs
  *_gradcheck, *_test     the reference's gradient checks and invariance tests (src/*.cpp)
  text_train              the reference training driver: checkpoint load, doc-masked windows, training epoch,
                          evaluation pass, checkpoint save
"""
import json
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "engine")
FIX = os.path.join(ROOT, "tests", "golden", "text_train")


def run(name, *args, cwd=None, timeout=600):
    exe = os.path.join(BIN, name)
    assert os.path.isfile(exe), f"{exe} is missing: build it with `make -C oracle` where the reference sources are"
    p = subprocess.run([exe, *args], cwd=cwd, capture_output=True, text=True, timeout=timeout)
    return p.returncode, (p.stdout + p.stderr).replace("\r", "\n")


def assert_clean(name, code, out):
    tail = "\n".join(out.strip().splitlines()[-25:])
    assert code == 0, f"{name} exited {code}:\n{tail}"
    assert "❌" not in out and "FAIL" not in out, f"{name} reported a failure:\n{tail}"


@pytest.mark.gpu
def test_engine_check_every_virtual_against_reference_cpu_engine():
    code, out = run("engine_check", "--verbose")
    print("\n".join(out.strip().splitlines()[-5:]))
    assert_clean("engine_check", code, out)
    m = re.search(r"engine_check: (\d+) cases, (\d+) failed", out)
    assert m and int(m.group(1)) >= 140 and int(m.group(2)) == 0


@pytest.mark.gpu
def test_engine_check_other_seed():
    code, out = run("engine_check", "--seed", "12345")
    assert_clean("engine_check", code, out)


@pytest.mark.gpu
@pytest.mark.parametrize("seed", ["7", "4242"])
def test_reference_gpt_model_agrees_on_both_engines(seed):
    """oracle/model_check.cpp: the reference's unchanged GPTModel (learned / sinusoidal / ALiBi / rotary positions, GeLU and
    SwiGLU, LayerNorm and RMSNorm, with and without document ids) on the reference CpuEngine and on the drop-in CUDA
    engine from the same seeded weights: logits, loss and every parameter gradient.  It takes the place of running the
    reference's gpt_gradcheck (weights from std::random_device against fp32 central differences: it fails about one
    run in three on the reference's own CPU engine) until it happens to pass."""
    code, out = run("model_check", "--seed", seed)
    assert_clean("model_check", code, out)
    m = re.search(r"model_check: (\d+) cases, (\d+) failed", out)
    assert m and int(m.group(1)) >= 21 and int(m.group(2)) == 0


REFERENCE_PROGRAMS = [
    ("attn_gradcheck", []),
    ("doc_attn_test", []),
    ("rmsnorm_gradcheck", []),
    ("softmax_gradcheck", []),
    ("swiglu_gradcheck", []),
    ("matmul_probe", []),
]


@pytest.mark.gpu
@pytest.mark.parametrize("name,args", REFERENCE_PROGRAMS, ids=[n + "".join("_" + a.strip("-") for a in a_) for n, a_ in REFERENCE_PROGRAMS])
def test_reference_program_passes_on_cuda_engine(name, args):
    code, out = run(name, "--cuda", *args)
    assert_clean(name, code, out)
    assert "CUDA" in out, f"{name} did not report the CUDA engine:\n{out[:400]}"


def _driver(tmp_path, *extra):
    exp = json.load(open(os.path.join(FIX, "expected.json")))
    for f in ("corpus.txt", "vocab.json", "start.bin"):
        dst = tmp_path / f
        if not dst.exists():
            dst.write_bytes(open(os.path.join(FIX, f), "rb").read())
    code, out = run("text_train", "corpus.txt", "--vocab", "vocab.json", *exp["model_args"], "--resume", "start.bin", *extra,
                    cwd=str(tmp_path), timeout=900)
    assert code == 0, out[-2000:]
    avg = [float(v) for v in re.findall(r"avg_loss=([0-9.]+)", out)]
    test = [float(v) for v in re.findall(r"test_loss=([0-9.]+)", out)]
    return exp, avg, test, out


@pytest.mark.gpu
def test_reference_training_driver_evaluation_pass_matches_cpu_engine(tmp_path):
    """Checkpoint load + forward + sparse cross-entropy over the whole corpus with the weights frozen (lr 0):
    the CUDA engine must print the loss the reference CPU engine printed (4 decimals in the log)."""
    exp, avg, test, out = _driver(tmp_path, "--cuda", "--save", "out.bin", "--test-file", "corpus.txt", "--lr", "0")
    assert "CUDA" in out
    assert test and abs(test[-1] - exp["eval_loss"]) <= 2e-4, (test, exp["eval_loss"])
    # the same run on the box's own CPU engine, live
    _, _, test_cpu, _ = _driver(tmp_path, "--save", "out_cpu.bin", "--test-file", "corpus.txt", "--lr", "0")
    assert abs(test[-1] - test_cpu[-1]) <= 2e-4
    # lr 0 leaves every parameter untouched: the checkpoint written through to_matrix equals the CPU engine's, byte for byte
    assert (tmp_path / "out.bin").read_bytes() == (tmp_path / "out_cpu.bin").read_bytes()


@pytest.mark.gpu
def test_reference_training_driver_epoch_matches_cpu_engine(tmp_path):
    """One AdamW epoch from the same checkpoint.  The driver shuffles windows from std::random_device, so
    runs differ a little even on one engine: the CUDA epoch loss must fall inside the CPU runs' spread
    widened by 1 %."""
    exp, avg, _, out = _driver(tmp_path, "--cuda", "--save", "out.bin", "--lr", "0.001")
    lo, hi = min(exp["train_loss"]), max(exp["train_loss"])
    assert avg and lo * 0.99 <= avg[-1] <= hi * 1.01, (avg, exp["train_loss"])
    # resume from the checkpoint the CUDA run wrote, on the CPU engine: the loss keeps falling from there
    for f in ("out.bin",):
        (tmp_path / "start.bin").write_bytes((tmp_path / f).read_bytes())
    _, avg2, _, _ = _driver(tmp_path, "--save", "out2.bin", "--lr", "0.001")
    assert avg2[-1] < avg[-1]


def test_cuda_engine_programs_do_not_fall_back_to_cpu():
    """Without a GPU a --cuda run must stop with an error, never continue on the CPU engine."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    exe = os.path.join(BIN, "gpt_gradcheck")
    if not os.path.isfile(exe):
        pytest.skip("oracle/_ref/engine is not built here")
    code, out = run("gpt_gradcheck", "--cuda")
    assert code != 0 and "CUDA" in out
