"""The fused training step driven from C++ through the reference's own API — Model::add<B200GPTModel>,
B200CrossEntropy, FusedAdamW / FusedMuon : nn::Optimizer, save_model — by neuralnet.cpp_b200/engine/fused_train
(compiled against the unmodified reference headers where the reference tree is present), against golden vectors of
the reference CPU engine: fp32 check mode within 1e-5, bf16 tensor-core mode within 1e-2."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import gpt_oracle as go
from oracle import ref_runner as rr
from tests.golden_io import global_rel_err, key_bias_indices, load_gpt_case, rel_err

pytestmark = pytest.mark.gpu

FUSED = os.path.join(entry.PKG_DIR, "engine", "build", "fused_train")


def _need_binary():
    if not os.path.isfile(FUSED):
        pytest.skip("fused_train was not built (make -C neuralnet.cpp_b200/engine REF=<reference tree>)")


def _run_case(name, precision, extra=()):
    case = load_gpt_case(name)
    out = rr.run_binary([FUSED, "run"], case["cfg"], case["params"], case["batches"],
                        extra_args=["--precision", str(precision)] + list(extra), dump_grads=True, dump_logits=True, **case["kw"])
    return case, out


@pytest.mark.parametrize("name", ["ln_gelu_learned", "rms_swiglu_alibi_accum", "docs_muon", "rms_swiglu_sin_clip"])
def test_cpp_host_check_mode_matches_reference(name):
    _need_binary()
    case, out = _run_case(name, 0)
    skip = key_bias_indices(case["cfg"])
    assert rel_err(out["logits"], case["logits"]) < 1e-5          # (vocab, tokens): the reference's own layout
    assert rel_err(out["losses"], case["losses"]) < 1e-5
    assert global_rel_err(out["grads"], case["grads"], skip) < 1e-5
    assert global_rel_err(out["params"], case["final"], skip) < 1e-5


@pytest.mark.parametrize("name", ["tile_rms_swiglu_alibi", "tile_docs_learned", "docs_muon"])
def test_cpp_host_bf16_mode_matches_reference(name):
    _need_binary()
    case, out = _run_case(name, 1)
    skip = key_bias_indices(case["cfg"])
    assert rel_err(out["losses"], case["losses"]) < 1e-2
    assert rel_err(out["logits"], case["logits"]) < 2e-2
    assert global_rel_err(out["params"], case["final"], skip) < 1e-2


def test_cpp_host_save_model_is_the_reference_file():
    """save_model on a Model holding the fused layer writes the v4 file the reference reads: byte-identical to the file
    this repository's Python writer (pinned against reference-written files) makes of the same parameters, and the
    reference CPU engine, started from those parameters, continues with the losses the fused run would have."""
    _need_binary()
    nnb = entry.load_package()
    from neuralnet_cpp_b200 import checkpoint
    case = load_gpt_case("rms_swiglu_alibi_accum")
    cfg = case["cfg"]
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "model.bin")
        _, out = _run_case("rms_swiglu_alibi_accum", 0, extra=["--save", path])
        spec, buf, off = checkpoint.read_model_file(path)
        mats, tok = checkpoint.split_matrices(buf, off, [(r, c) for _, r, c in go.param_shapes(cfg)])
        assert tok == b""
        for got, want in zip(mats, out["params"]):
            assert np.array_equal(got, want)
        tcfg = nnb.GptConfig(cfg.vocab, cfg.d_model, cfg.heads, cfg.layers, cfg.d_ff, cfg.seq, cfg.batch, cfg.act, cfg.norm, cfg.pos, 0)
        ref_path = os.path.join(td, "py.bin")
        checkpoint.write_model_file(ref_path, checkpoint.spec_of_config(tcfg), out["params"], b"")
        assert open(path, "rb").read() == open(ref_path, "rb").read()
    if rr.available():
        mbs = go.make_batches(cfg, 1, seed=9, dist="zipf")
        ref = rr.run_reference(cfg, out["params"], mbs, steps=1, lr=1e-3, wd=0.01, skip_params=True)
        again = rr.run_binary([FUSED, "run"], cfg, out["params"], mbs, extra_args=["--precision", "0"], steps=1, lr=1e-3, wd=0.01,
                              skip_params=True)
        assert rel_err(again["losses"], ref["losses"]) < 1e-5


def test_cpp_host_forward_step_and_generate_match_reference():
    """B200GPTModel::forward_step / ::generate (key/value cache) through the C++ host against the reference's
    GPTModel::forward_step / ::generate golden vectors."""
    _need_binary()
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode.npz"))
    for name in ("ln_gelu_learned", "rms_swiglu_alibi", "rms_swiglu_rope"):
        cfg = go.GptConfig(*[int(v) for v in z[name + "_cfg"]])
        params = go.init_params(cfg, 42, std=0.2)
        mbs = go.make_batches(cfg, 1, seed=1)
        out = rr.run_binary([FUSED, "run"], cfg, params, mbs, extra_args=["--precision", "0"], steps=0, lr=1e-3, skip_params=True,
                            decode_tokens=z[name + "_tokens"], decode_steps=cfg.seq)
        assert rel_err(out["decode_logits"], z[name + "_logits"]) < 1e-5
        gen = rr.run_binary([FUSED, "run"], cfg, params, mbs, extra_args=["--precision", "0"], steps=0, lr=1e-3, skip_params=True,
                            decode_tokens=z[name + "_tokens"][:10], generate=cfg.seq + 6)
        assert np.array_equal(gen["generated"], z[name + "_generated"])


def test_cpp_host_bench_mode_runs():
    """The benchmark loop of the C++ host on a shallow copy of the benchmark model: one JSON line, finite loss."""
    _need_binary()
    import json
    r = subprocess.run([FUSED, "bench", "--steps", "2", "--warmup", "1", "--layers", "2", "--batch", "4"], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["host"] == "cpp" and line["ms_per_step"] > 0 and line["gpu_launches"] > 0 and np.isfinite(line["last_loss"])
