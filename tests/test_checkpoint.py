"""Checkpoints either side of the training step: the reference's model file (format v4) read and written from the
fused trainer, and the trainer's own full training state (parameters, optimizer moments, step).

The reference-written file of the fixture (tests/golden/text_train/start.bin, made by the reference driver on its
CPU engine) is the golden vector for the format."""
import os
import subprocess

import numpy as np
import pytest

import __graft_entry__ as entry

ROOT = entry.ROOT
FIX = os.path.join(ROOT, "tests", "golden", "text_train")


def _ck():
    entry.load_package()
    from neuralnet_cpp_b200 import checkpoint
    return checkpoint


def _fixture_shapes():
    from oracle import gpt_oracle as go
    cfg = go.GptConfig(vocab=414, d_model=64, heads=4, layers=2, d_ff=128, seq=32, batch=8, act=1, norm=1, pos=2)
    return cfg, [(r, c) for _, r, c in go.param_shapes(cfg)]


def test_reference_model_file_round_trips_byte_for_byte(tmp_path):
    ck = _ck()
    spec, buf, off = ck.read_model_file(os.path.join(FIX, "start.bin"))
    assert spec == {"type": 3, "layer_dims": [], "d_model": 64, "num_heads": 4, "d_ff": 128, "num_layers": 2, "patch_size": 0,
                    "vocab_size": 414, "seq_len": 32, "pos_encoding": 2, "activation": 1, "norm_type": 1}
    _, shapes = _fixture_shapes()
    mats, tok = ck.split_matrices(buf, off, shapes)
    assert len(mats) == 32 and tok == open(os.path.join(FIX, "vocab.json"), "rb").read()
    out = tmp_path / "copy.bin"
    ck.write_model_file(str(out), spec, mats, tok)
    assert out.read_bytes() == bytes(buf)


def test_reference_model_file_rejects_wrong_shapes_and_foreign_files(tmp_path):
    ck = _ck()
    spec, buf, off = ck.read_model_file(os.path.join(FIX, "start.bin"))
    _, shapes = _fixture_shapes()
    bad = list(shapes)
    bad[1] = (64, 65)
    with pytest.raises(ValueError, match="Matrix shape mismatch"):
        ck.split_matrices(buf, off, bad)
    junk = tmp_path / "junk.bin"
    junk.write_bytes(b"not a model file at all")
    with pytest.raises(ValueError, match="not a neuralnet.cpp model file"):
        ck.read_model_file(str(junk))


def test_key_value_record_serialisation():
    ck = _ck()
    fields = [("type", 3), ("layer_dims", [784, 128, 10]), ("name", "gpt"), ("d_model", 2 ** 40 + 5)]
    assert ck._parse_kv(ck._serialize_kv(fields)) == dict(fields)


def test_training_state_file_round_trip(tmp_path):
    ck = _ck()
    r = np.random.default_rng(0)
    arenas = {"params": r.standard_normal(1000).astype(np.float32), "m": r.standard_normal(1000).astype(np.float32),
              "v": r.random(1000).astype(np.float32)}
    p = str(tmp_path / "state.bin")
    ck.save_training_state(p, arenas, 17, [1, 2, 3])
    got, step, cfg = ck.load_training_state(p)
    assert step == 17 and cfg == [1, 2, 3] and all(np.array_equal(got[k], arenas[k]) for k in arenas)


def _trainer(nnb, precision, **kw):
    cfg = nnb.GptConfig(414, 64, 4, 2, 128, 32, 8, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_ALIBI, precision)
    return nnb.GptTrainer(cfg, lr=1e-3, weight_decay=0.01, **kw)


def _batch(seed):
    r = np.random.default_rng(seed)
    ids = r.integers(0, 414, (8, 33))
    return ids[:, :-1].reshape(-1).astype(np.int32), ids[:, 1:].reshape(-1).astype(np.int32)


@pytest.mark.gpu
def test_fused_trainer_loads_and_writes_the_reference_model_file(tmp_path):
    """The weights of the reference-written file land where the fused step expects them (loss equal to the oracle's
    on the same matrices), and the file written back is byte-identical, tokenizer included; the reference's own
    loader accepts it."""
    from oracle import gpt_oracle as go
    from tests import gpu_util
    nnb = gpu_util.nnb
    tr = _trainer(nnb, nnb.FP32)
    tok = tr.load_reference_checkpoint(os.path.join(FIX, "start.bin"))
    assert len(tok) == os.path.getsize(os.path.join(FIX, "vocab.json"))
    x, y = _batch(1)
    tr.forward(x)
    tr.loss_and_grad(y, None, 1.0)
    got = float(tr.loss_tensor().item())
    ocfg, _ = _fixture_shapes()
    model = go.GptOracle(ocfg, tr.get_params())
    logits = model.forward(x.astype(np.float32).reshape(8, 32))
    want, _ = go.ce_forward_sparse(logits, y.astype(np.float32), None, 414)
    assert abs(got - float(want)) <= 1e-5 * abs(float(want)), (got, want)
    out = tmp_path / "back.bin"
    tr.save_reference_checkpoint(str(out), tok)
    assert out.read_bytes() == open(os.path.join(FIX, "start.bin"), "rb").read()
    wrong = nnb.GptTrainer(nnb.GptConfig(414, 64, 4, 3, 128, 32, 8, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_ALIBI, nnb.FP32))
    with pytest.raises(ValueError, match="num_layers"):
        wrong.load_reference_checkpoint(os.path.join(FIX, "start.bin"))


@pytest.mark.gpu
def test_reference_driver_resumes_from_a_checkpoint_the_fused_trainer_wrote(tmp_path):
    """Three AdamW steps on the fused trainer, written as a reference model file: the reference driver (its CPU
    engine) resumes from it and evaluates."""
    import json
    import re
    from tests import gpu_util
    nnb = gpu_util.nnb
    tr = _trainer(nnb, nnb.FP32)        # the fixture's vocabulary (414) is not a multiple of 8: bf16 mode refuses it
    tok = tr.load_reference_checkpoint(os.path.join(FIX, "start.bin"))
    for s in range(3):
        x, y = _batch(10 + s)
        tr.forward(x)
        tr.loss_and_grad(y, None, 1.0)
        tr.backward()
        tr.optimizer_step()
    for f in ("corpus.txt", "vocab.json"):
        (tmp_path / f).write_bytes(open(os.path.join(FIX, f), "rb").read())
    tr.save_reference_checkpoint(str(tmp_path / "fused.bin"), tok)
    exp = json.load(open(os.path.join(FIX, "expected.json")))
    exe = os.path.join(ROOT, "oracle", "_ref", "engine", "text_train")
    assert os.path.isfile(exe), "build oracle/_ref with `make -C oracle` where the reference sources are"
    p = subprocess.run([exe, "corpus.txt", "--vocab", "vocab.json", *exp["model_args"], "--resume", "fused.bin", "--save", "o.bin",
                        "--test-file", "corpus.txt", "--lr", "0"], cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    out = (p.stdout + p.stderr).replace("\r", "\n")
    assert p.returncode == 0, out[-1500:]
    test = [float(v) for v in re.findall(r"test_loss=([0-9.]+)", out)]
    # three steps on random tokens barely move a model trained on the corpus: the loss stays near the fixture's
    assert test and abs(test[-1] - exp["eval_loss"]) < 0.5, (test, exp["eval_loss"])


@pytest.mark.gpu
def test_evaluation_pass_weights_batches_by_valid_targets():
    """GptTrainer.evaluate against the oracle on the fixture checkpoint: two batches with different numbers of masked
    targets, averaged as the reference driver averages its test loss (text_train.cpp:1455-1463)."""
    from oracle import gpt_oracle as go
    from tests import gpu_util
    nnb = gpu_util.nnb
    tr = _trainer(nnb, nnb.FP32)
    tr.load_reference_checkpoint(os.path.join(FIX, "start.bin"))
    ocfg, _ = _fixture_shapes()
    model = go.GptOracle(ocfg, tr.get_params())
    r = np.random.default_rng(5)
    batches, num, den = [], 0.0, 0.0
    for keep in (0.9, 0.4):
        x, y = _batch(int(keep * 10))
        mask = (r.random(x.size) < keep).astype(np.float32)
        batches.append((x, y, mask))
        loss, _ = go.ce_forward_sparse(model.forward(x), y.astype(np.float32), mask, 414)
        num += float(loss) * float(mask.sum())
        den += float(mask.sum())
    before = [g.copy() for g in tr.get_grads()]
    got = tr.evaluate(batches)
    assert abs(got - num / den) <= 1e-5 * abs(num / den), (got, num / den)
    assert all(np.array_equal(a, b) for a, b in zip(before, tr.get_grads()))


@pytest.mark.gpu
@pytest.mark.parametrize("muon", [False, True])
def test_training_state_resume_is_exact_in_check_mode(tmp_path, muon):
    """Save after three steps, run two more; a fresh trainer that loads the state runs the same two steps to the
    same losses and parameters, bit for bit (fp32 check mode has no atomics)."""
    from tests import gpu_util
    nnb = gpu_util.nnb

    def steps(tr, first, n):
        losses = []
        for s in range(first, first + n):
            x, y = _batch(100 + s)
            tr.forward(x)
            tr.loss_and_grad(y, None, 1.0)
            tr.backward()
            losses.append(float(tr.loss_tensor().item()))
            tr.optimizer_step(clip=1.0)
        return losses

    a = _trainer(nnb, nnb.FP32, muon=muon)
    a.init_params_normal(seed=3)
    steps(a, 0, 3)
    a.save_training_state(str(tmp_path / "state.bin"))
    want = steps(a, 3, 2)
    b = _trainer(nnb, nnb.FP32, muon=muon)
    b.load_training_state(str(tmp_path / "state.bin"))
    assert b.t == 3
    got = steps(b, 3, 2)
    assert got == want
    assert all(np.array_equal(p, q) for p, q in zip(a.get_params(), b.get_params()))
    other = _trainer(nnb, nnb.FP32, muon=not muon)
    with pytest.raises(ValueError):
        other.load_training_state(str(tmp_path / "state.bin"))
