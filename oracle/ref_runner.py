"""TEST INFRASTRUCTURE — runs the compiled reference CPU engine harness (oracle/_ref/ref_gpt).

Writes the binary input file ``oracle/ref_harness.cpp`` documents, executes the binary and parses
its output.  Used to generate the golden vectors, to pin the numpy restatement and as the timed
CPU baseline.  The product never imports this module.
"""
from __future__ import annotations

import os
import struct
import subprocess
import tempfile
from typing import List, Optional

import numpy as np

from . import gpt_oracle as go

HERE = os.path.dirname(os.path.abspath(__file__))
REF_BIN = os.path.join(HERE, "_ref", "ref_gpt")


def available() -> bool:
    return os.path.isfile(REF_BIN) and os.access(REF_BIN, os.X_OK)


def write_input(path, cfg: go.GptConfig, params, micro_batches, *, steps, accum=1, lr=1e-3, wd=0.01,
                optimizer=go.OPT_ADAMW, muon_lr=0.02, clip=None, cosine=False, warmup=0, total_steps=1, min_lr=0.0,
                dump_grads=False, dump_logits=False, skip_params=False, decode_tokens=None, decode_steps=0, generate=0):
    """Writes the binary run description oracle/ref_harness.cpp documents."""
    shapes = go.param_shapes(cfg)
    use_doc = micro_batches[0].get("doc_ids") is not None
    I = np.zeros(32, np.int32)
    I[:23] = [cfg.vocab, cfg.d_model, cfg.heads, cfg.layers, cfg.d_ff, cfg.seq, cfg.batch, cfg.act,
              cfg.norm, cfg.pos, int(use_doc), steps, accum, optimizer, int(clip is not None),
              int(cosine), warmup, total_steps, int(dump_grads), int(dump_logits), int(skip_params),
              int(decode_steps), int(generate)]
    F = np.zeros(16, np.float32)
    F[:5] = [lr, wd, clip if clip is not None else 0.0, min_lr, muon_lr]
    with open(path, "wb") as f:
        f.write(struct.pack("<I", 0x3242424E))
        f.write(I.tobytes())
        f.write(F.tobytes())
        f.write(struct.pack("<i", len(shapes)))
        for p, (_, r, c) in zip(params, shapes):
            f.write(struct.pack("<ii", r, c))
            f.write(np.ascontiguousarray(p, np.float32).reshape(r, c).tobytes())
        assert len(micro_batches) >= steps * accum
        for mb in micro_batches[:steps * accum]:
            f.write(np.asarray(mb["tokens"], np.int32).tobytes())
            f.write(np.asarray(mb["labels"], np.int32).tobytes())
            f.write(np.asarray(mb["mask"], np.float32).tobytes())
            if use_doc:
                f.write(np.asarray(mb["doc_ids"], np.int32).tobytes())
        if decode_tokens is not None:
            ids = np.asarray(decode_tokens, np.int32)
            f.write(struct.pack("<i", ids.size))
            f.write(ids.tobytes())


def parse_output(raw: bytes, cfg: go.GptConfig, *, steps, accum=1, dump_grads=False, dump_logits=False, skip_params=False,
                 decode_steps=0, generate=0):
    """dict(losses, grads|None, logits|None, params|None, seconds[, decode_logits, generated]) from the output file of a run."""
    shapes = go.param_shapes(cfg)
    off = 0

    def take(n, dt=np.float32):
        nonlocal off
        a = np.frombuffer(raw, dt, n, off).copy()
        off += a.nbytes
        return a

    out = {"losses": take(steps * accum), "grads": None, "logits": None, "params": None}
    if dump_grads:
        out["grads"] = [take(rr * cc).reshape(rr, cc) for _, rr, cc in shapes]
    if dump_logits:
        out["logits"] = take(cfg.vocab * cfg.tokens).reshape(cfg.vocab, cfg.tokens)
    if not skip_params:
        out["params"] = [take(rr * cc).reshape(rr, cc) for _, rr, cc in shapes]
    out["seconds"] = take(steps, np.float64)
    if decode_steps:
        out["decode_logits"] = take(decode_steps * cfg.vocab).reshape(decode_steps, cfg.vocab)
    if generate:
        n = int(take(1, np.int32)[0])
        out["generated"] = take(n, np.int32)
    assert off == len(raw), (off, len(raw))
    return out


def run_binary(binary, cfg: go.GptConfig, params, micro_batches, extra_args=(), threads: Optional[int] = None, timeout=3600,
               **kw):
    """Runs `binary in.bin out.bin [extra_args]` on the run described by the keywords of write_input."""
    io_kw = dict(steps=kw["steps"], accum=kw.get("accum", 1), dump_grads=kw.get("dump_grads", False),
                 dump_logits=kw.get("dump_logits", False), skip_params=kw.get("skip_params", False),
                 decode_steps=kw.get("decode_steps", 0), generate=kw.get("generate", 0))
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
        write_input(fin, cfg, params, micro_batches, **kw)
        cmd = list(binary) + [fin, fout] + list(extra_args)
        if threads:
            cmd = ["taskset", "-c", "0-%d" % (threads - 1)] + cmd
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        if r.returncode != 0:
            raise RuntimeError("%s failed (%d): %s" % (os.path.basename(binary[-1] if len(binary) == 1 else binary[0]), r.returncode, r.stderr[-2000:]))
        raw = open(fout, "rb").read()
    out = parse_output(raw, cfg, **io_kw)
    out["stderr"] = r.stderr
    return out


def run_reference(cfg: go.GptConfig, params, micro_batches, *, threads: Optional[int] = None, timeout=3600, **kw):
    """The run on the reference CPU engine (oracle/_ref/ref_gpt).  Keywords: those of write_input.
    Returns dict(losses, grads|None, logits|None, params|None, seconds)."""
    if not available():
        raise RuntimeError("reference harness not built: run `make -C oracle REF=...` where the reference tree is present")
    return run_binary([REF_BIN], cfg, params, micro_batches, threads=threads, timeout=timeout, **kw)
