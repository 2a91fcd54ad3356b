"""Regenerates tests/golden/*.npz from the unmodified reference CPU engine.

Run where the reference tree is present:  make -C oracle && python tests/golden/make_golden.py
The vectors are outputs of oracle/_ref/ref_gpt and oracle/_ref/ref_prims (the reference's CpuEngine,
GPTModel, CrossEntropyLoss, AdamW, Muon) on seeded synthetic inputs; inputs are stored with them.
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import gpt_oracle as go  # noqa: E402
from oracle import ref_runner as rr  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))

# name -> (config, training keywords, token distribution, packed documents)
CASES = {
    "ln_gelu_learned": (go.GptConfig(64, 32, 4, 2, 64, 16, 3, go.ACT_GELU, go.NORM_LAYER, go.POS_LEARNED),
                        dict(steps=4, lr=1e-3, wd=0.01), "uniform", False),
    "rms_swiglu_sin_clip": (go.GptConfig(96, 48, 6, 2, 80, 12, 4, go.ACT_SWIGLU, go.NORM_RMS, go.POS_SINUSOIDAL),
                            dict(steps=4, lr=6e-4, wd=0.01, clip=1.0), "zipf", False),
    "rms_swiglu_alibi_accum": (go.GptConfig(80, 32, 4, 2, 64, 16, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ALIBI),
                               dict(steps=3, accum=2, lr=1e-3, wd=0.01, cosine=True, warmup=1, total_steps=3,
                                    min_lr=1e-4), "zipf", False),
    "docs_muon": (go.GptConfig(72, 32, 4, 2, 48, 24, 3, go.ACT_SWIGLU, go.NORM_RMS, go.POS_LEARNED),
                  dict(steps=3, lr=1e-3, wd=0.01, optimizer=go.OPT_MUON_SPLIT, muon_lr=0.02), "zipf", True),
    # head_dim 64 / 128-wide tiles: shapes the tensor-core kernels tile without remainder
    "tile_rms_swiglu_alibi": (go.GptConfig(256, 128, 2, 1, 256, 128, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ALIBI),
                              dict(steps=3, accum=2, lr=1e-3, wd=0.01), "zipf", False),
    "tile_docs_learned": (go.GptConfig(256, 128, 2, 1, 192, 256, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_LEARNED),
                          dict(steps=2, lr=1e-3, wd=0.01, clip=1.0), "zipf", True),
    # rotary position encoding on Q and K (RotaryEmbedding, compute_layer.hpp:876-988)
    "rms_swiglu_rope": (go.GptConfig(80, 32, 4, 2, 64, 16, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ROPE),
                        dict(steps=3, lr=1e-3, wd=0.01, clip=1.0), "zipf", False),
    "tile_rope_docs": (go.GptConfig(256, 128, 2, 1, 256, 128, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ROPE),
                       dict(steps=2, accum=2, lr=1e-3, wd=0.01), "zipf", True),
}
# Full-width cases (BASELINE configurations 2, 3 and 4 at the model shapes the benchmark runs): too large to
# store whole, so each keeps per-micro-batch losses, a fixed sample of the first logits, and per tensor the
# L2 norm plus a fixed sample (sample_indices) of the first-step gradient and of the final parameters.
FULL_CASES = {
    # configuration 2 at full size, two optimizer steps
    "full_c2": (go.GptConfig(4096, 384, 6, 6, 1024, 256, 32, go.ACT_SWIGLU, go.NORM_RMS, go.POS_SINUSOIDAL),
                dict(steps=2, lr=6e-4, wd=0.01, clip=1.0), "zipf", False),
    # configuration 3 at full model shape, micro-batch 2 x accumulation 2, cosine schedule
    "full_c3": (go.GptConfig(8192, 768, 12, 12, 2048, 1024, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ALIBI),
                dict(steps=2, accum=2, lr=6e-4, wd=0.01, cosine=True, warmup=1, total_steps=4, min_lr=6e-5),
                "zipf", False),
    # configuration 4 at full width, two layers, one packed row of geometric(300) documents, Muon split
    "full_c4": (go.GptConfig(16384, 1024, 16, 2, 2816, 2048, 1, go.ACT_SWIGLU, go.NORM_RMS, go.POS_LEARNED),
                dict(steps=2, lr=1e-3, wd=0.01, optimizer=go.OPT_MUON_SPLIT, muon_lr=0.02), "zipf", True),
}
SAMPLE = 4096


def sample_indices(size, k=SAMPLE):
    """Fixed, well-spread flat indices into a tensor of `size` elements (all of them when size <= k)."""
    if size <= k:
        return np.arange(size, dtype=np.int64)
    return (np.arange(k, dtype=np.int64) * 7919003) % size


# BASELINE configuration 1 (tiny GPT, 20 steps): only losses and per-tensor norms are stored
C1 = go.GptConfig(512, 128, 4, 2, 512, 128, 8, go.ACT_GELU, go.NORM_LAYER, go.POS_LEARNED)


def pack_batches(mbs):
    d = {"tokens": np.stack([m["tokens"] for m in mbs]), "labels": np.stack([m["labels"] for m in mbs]),
         "mask": np.stack([m["mask"] for m in mbs])}
    if mbs[0]["doc_ids"] is not None:
        d["doc_ids"] = np.stack([m["doc_ids"] for m in mbs])
    return d


def gpt_cases(only=None):
    for name, (cfg, kw, dist, docs) in CASES.items():
        if only and name not in only:
            continue
        params = go.init_params(cfg, 42)
        mbs = go.make_batches(cfg, kw["steps"] * kw.get("accum", 1), seed=1, dist=dist, docs=docs)
        ref = rr.run_reference(cfg, params, mbs, dump_grads=True, dump_logits=True, **kw)
        arrays = {"cfg": np.array(list(vars(cfg).values()), np.int64),
                  "kw_keys": np.array(list(kw.keys())), "kw_vals": np.array([float(v) for v in kw.values()]),
                  "losses": ref["losses"], "logits": ref["logits"]}
        arrays.update(pack_batches(mbs))
        # initial parameters are regenerated by init_params(cfg, 42); their checksum guards RNG drift
        arrays["p0_checksum"] = np.array([float(sum(np.abs(p.astype(np.float64)).sum() for p in params))])
        for i, (g, p1) in enumerate(zip(ref["grads"], ref["params"])):
            arrays[f"g_{i}"], arrays[f"p1_{i}"] = g, p1
        np.savez_compressed(os.path.join(OUT, f"gpt_{name}.npz"), **arrays)
        print(name, "losses", ref["losses"])


def full_cases(only=None):
    for name, (cfg, kw, dist, docs) in FULL_CASES.items():
        if only and name not in only:
            continue
        params = go.init_params(cfg, 42)
        mbs = go.make_batches(cfg, kw["steps"] * kw.get("accum", 1), seed=1, dist=dist, docs=docs)
        ref = rr.run_reference(cfg, params, mbs, dump_grads=True, dump_logits=True, timeout=6 * 3600, **kw)
        lg = ref["logits"].T.reshape(-1)                       # token-major (tokens, vocab)
        arrays = {"cfg": np.array(list(vars(cfg).values()), np.int64),
                  "kw_keys": np.array(list(kw.keys())), "kw_vals": np.array([float(v) for v in kw.values()]),
                  "losses": ref["losses"], "logits_sample": lg[sample_indices(lg.size, 4 * SAMPLE)],
                  "logits_absmax": np.array([np.abs(lg).max()]),
                  "seconds": ref["seconds"]}
        arrays.update(pack_batches(mbs))
        arrays["p0_checksum"] = np.array([float(sum(np.abs(p.astype(np.float64)).sum() for p in params))])
        arrays["g_norms"] = np.array([np.linalg.norm(g.astype(np.float64)) for g in ref["grads"]])
        arrays["p1_norms"] = np.array([np.linalg.norm(p.astype(np.float64)) for p in ref["params"]])
        arrays["g_absmax"] = np.array([np.abs(g).max() for g in ref["grads"]])
        for i, (g, p1) in enumerate(zip(ref["grads"], ref["params"])):
            idx = sample_indices(g.size)
            arrays[f"g_{i}"], arrays[f"p1_{i}"] = g.reshape(-1)[idx], p1.reshape(-1)[idx]
        np.savez_compressed(os.path.join(OUT, f"gpt_{name}.npz"), **arrays)
        print(name, "losses", ref["losses"], "s/step", ref["seconds"], flush=True)


# Incremental inference with a key/value cache: GPTModel::forward_step over a token list (logits of every step) and
# GPTModel::generate at temperature 0 (prompt 10 tokens, more new tokens than the window has room for, so the sliding
# window rebuild runs).  Weights N(0, 0.2) so that the arg max of the logits is well separated.
DECODE_CASES = {
    "ln_gelu_learned": go.GptConfig(96, 48, 6, 2, 80, 16, 1, go.ACT_GELU, go.NORM_LAYER, go.POS_LEARNED),
    "rms_swiglu_sin": go.GptConfig(96, 48, 6, 2, 80, 16, 1, go.ACT_SWIGLU, go.NORM_RMS, go.POS_SINUSOIDAL),
    "rms_swiglu_alibi": go.GptConfig(128, 64, 4, 3, 96, 24, 1, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ALIBI),
    "rms_swiglu_rope": go.GptConfig(128, 64, 4, 2, 96, 24, 1, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ROPE),
}


def decode_cases():
    arrays = {}
    for name, cfg in DECODE_CASES.items():
        params = go.init_params(cfg, 42, std=0.2)
        rng = np.random.default_rng(77)
        tokens = rng.integers(0, cfg.vocab, cfg.seq).astype(np.int32)          # a full window of tokens, step by step
        mbs = go.make_batches(cfg, 1, seed=1)
        ref = rr.run_reference(cfg, params, mbs, steps=0, lr=1e-3, skip_params=True, decode_tokens=tokens,
                               decode_steps=cfg.seq)
        gen = rr.run_reference(cfg, params, mbs, steps=0, lr=1e-3, skip_params=True, decode_tokens=tokens[:10],
                               generate=cfg.seq + 6)
        arrays[name + "_cfg"] = np.array(list(vars(cfg).values()), np.int64)
        arrays[name + "_tokens"] = tokens
        arrays[name + "_logits"] = ref["decode_logits"]
        arrays[name + "_generated"] = gen["generated"]
        arrays[name + "_p0_checksum"] = np.array([float(sum(np.abs(p.astype(np.float64)).sum() for p in params))])
        print("decode", name, gen["generated"][:8], "...")
    np.savez_compressed(os.path.join(OUT, "decode.npz"), **arrays)


def c1_case():
    params = go.init_params(C1, 42)
    mbs = go.make_batches(C1, 20, seed=1, dist="uniform")
    ref = rr.run_reference(C1, params, mbs, steps=20, lr=1e-3, wd=0.01)
    arrays = {"cfg": np.array(list(vars(C1).values()), np.int64), "losses": ref["losses"],
              "p0_norms": np.array([np.linalg.norm(p.astype(np.float64)) for p in params]),
              "p1_norms": np.array([np.linalg.norm(p.astype(np.float64)) for p in ref["params"]]),
              "p1_lm_head_b": ref["params"][-1], "p1_ln_f_beta": ref["params"][-3],
              "p1_ln_f_gamma": ref["params"][-4]}
    arrays.update(pack_batches(mbs))
    np.savez_compressed(os.path.join(OUT, "gpt_c1_20steps.npz"), **arrays)
    print("c1 losses", ref["losses"], "s/step", ref["seconds"].mean())


def prim_case():
    rng = np.random.default_rng(2026)
    batch, M, N, K, D, C, NC, vocab = 3, 7, 7, 5, 6, 9, 11, 8
    alpha, inv_nv = 0.35, 1.0 / 9.0
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    A, B, V, G, P = f(batch * K, M), f(batch * K, N), f(batch * N, D), f(batch * M, D), f(batch * M, N)
    mask = np.where(np.arange(N)[None, :] <= np.arange(M)[:, None], 0.0, -np.inf).astype(np.float32)
    logits = f(C, NC)
    labels = rng.integers(0, C + 2, (1, NC)).astype(np.float32)     # some labels out of range
    cmask = (rng.random((1, NC)) > 0.25).astype(np.float32)
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "i"), os.path.join(td, "o")
        with open(fin, "wb") as fh:
            fh.write(np.array([batch, M, N, K, D, C, NC, vocab], np.int32).tobytes())
            fh.write(struct.pack("<ff", alpha, inv_nv))
            for a in (A, B, V, G, P, mask, logits, labels, cmask):
                fh.write(a.tobytes())
        subprocess.run([os.path.join(ROOT, "oracle", "_ref", "ref_prims"), fin, fout], check=True)
        raw = np.fromfile(fout, np.float32)
    shapes = [("m", (batch * M, 1)), ("l", (batch * M, 1)), ("O", (batch * M, D)), ("gradQ", (batch * K, M)),
              ("R", (batch * M, 1)), ("gradK", (batch * K, N)), ("gradV", (batch * K, N)), ("col_denom", (1, NC)),
              ("ce_grad", (C, NC)), ("loss_vec", (1, NC)), ("gathered", (NC, NC)), ("scattered", (C, NC)),
              ("rearranged", (K, batch * M))]
    arrays, off = {}, 0
    for n, s in shapes:
        k = int(np.prod(s))
        arrays["out_" + n] = raw[off:off + k].reshape(s)
        off += k
    assert off == raw.size
    arrays.update(A=A, B=B, V=V, G=G, P=P, mask=mask, logits=logits, labels=labels, cmask=cmask,
                  dims=np.array([batch, M, N, K, D, C, NC, vocab]), scal=np.array([alpha, inv_nv], np.float32))
    np.savez_compressed(os.path.join(OUT, "prims.npz"), **arrays)
    print("prims ok")


if __name__ == "__main__":
    which = sys.argv[1:] or ["prims", "gpt", "c1", "decode"]
    if "prims" in which:
        prim_case()
    if "gpt" in which:
        gpt_cases()
    named = [w for w in which if w in CASES]          # e.g. `make_golden.py rms_swiglu_rope` regenerates one case
    if named:
        gpt_cases(named)
    named = [w for w in which if w in FULL_CASES]     # hours of CPU time in total: only when named, or with `full`
    if named or "full" in which:
        full_cases(named or None)
    if "c1" in which:
        c1_case()
    if "decode" in which:
        decode_cases()
