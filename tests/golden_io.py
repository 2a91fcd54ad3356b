"""Loads the golden vectors under tests/golden/ (outputs of the reference CPU engine)."""
import os

import numpy as np

from oracle import gpt_oracle as go

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GPT_CASES = ["ln_gelu_learned", "rms_swiglu_sin_clip", "rms_swiglu_alibi_accum", "docs_muon",
             "tile_rms_swiglu_alibi", "tile_docs_learned", "rms_swiglu_rope", "tile_rope_docs"]
INT_KW = {"steps", "accum", "optimizer", "warmup", "total_steps"}


def load_gpt_case(name):
    z = np.load(os.path.join(GOLDEN, f"gpt_{name}.npz"))
    cfg = go.GptConfig(*[int(v) for v in z["cfg"]])
    kw = {}
    for k, v in zip(z["kw_keys"], z["kw_vals"]):
        k = str(k)
        kw[k] = int(v) if k in INT_KW else (bool(v) if k == "cosine" else float(v))
    n = kw["steps"] * kw.get("accum", 1)
    mbs = [{"tokens": z["tokens"][i], "labels": z["labels"][i], "mask": z["mask"][i],
            "doc_ids": z["doc_ids"][i] if "doc_ids" in z.files else None} for i in range(n)]
    params = go.init_params(cfg, 42)
    chk = float(sum(np.abs(p.astype(np.float64)).sum() for p in params))
    assert abs(chk - float(z["p0_checksum"][0])) <= 1e-9 * chk, "numpy RNG stream changed: regenerate goldens"
    k = len(go.param_shapes(cfg))
    return dict(cfg=cfg, kw=kw, batches=mbs, params=params, losses=z["losses"], logits=z["logits"],
                grads=[z[f"g_{i}"] for i in range(k)], final=[z[f"p1_{i}"] for i in range(k)])


FULL_CASES = ["full_c2", "full_c3", "full_c4"]


def sample_indices(size, k=4096):
    """The fixed flat indices tests/golden/make_golden.py sampled every tensor of a full-width case at."""
    if size <= k:
        return np.arange(size, dtype=np.int64)
    return (np.arange(k, dtype=np.int64) * 7919003) % size


def load_full_case(name):
    """A full-width case (BASELINE configurations 2, 3, 4 at the model shapes the benchmark runs): outputs of the
    reference CPU engine stored as per-micro-batch losses, a sample of the first logits, and per tensor the L2 norm and
    a 4096-element sample of the first-step gradient and of the final parameters."""
    z = np.load(os.path.join(GOLDEN, f"gpt_{name}.npz"))
    cfg = go.GptConfig(*[int(v) for v in z["cfg"]])
    kw = {}
    for k, v in zip(z["kw_keys"], z["kw_vals"]):
        k = str(k)
        kw[k] = int(v) if k in INT_KW else (bool(v) if k == "cosine" else float(v))
    n = kw["steps"] * kw.get("accum", 1)
    mbs = [{"tokens": z["tokens"][i], "labels": z["labels"][i], "mask": z["mask"][i],
            "doc_ids": z["doc_ids"][i] if "doc_ids" in z.files else None} for i in range(n)]
    params = go.init_params(cfg, 42)
    chk = float(sum(np.abs(p.astype(np.float64)).sum() for p in params))
    assert abs(chk - float(z["p0_checksum"][0])) <= 1e-9 * chk, "numpy RNG stream changed: regenerate goldens"
    k = len(go.param_shapes(cfg))
    return dict(cfg=cfg, kw=kw, batches=mbs, params=params, losses=z["losses"], logits_sample=z["logits_sample"],
                logits_absmax=float(z["logits_absmax"][0]), g_norms=z["g_norms"], p1_norms=z["p1_norms"],
                g_absmax=z["g_absmax"], grads=[z[f"g_{i}"] for i in range(k)], final=[z[f"p1_{i}"] for i in range(k)])


def sample_tensors(tensors):
    """Each tensor reduced to the sample the full-width goldens keep."""
    return [np.asarray(t).reshape(-1)[sample_indices(np.asarray(t).size)] for t in tensors]


def rel_err(a, b):
    """max |a-b| / max |b| — the relative norm the parity bar is stated in."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


def key_bias_indices(cfg):
    """Indices of the wk.b tensors.  Their gradient is analytically zero (softmax is invariant to a
    per-query shift of the scores), so both engines hold pure rounding noise there and Adam turns
    that noise into +-lr steps; they are excluded from parameter comparisons."""
    return {i for i, (n, _, _) in enumerate(go.param_shapes(cfg)) if n.endswith("wk.b")}


def global_rel_err(xs, refs, skip=()):
    """||x - ref||_2 / ||ref||_2 over all tensors concatenated (the parameter-parity figure)."""
    num = sum(float(((np.asarray(a, np.float64) - np.asarray(b, np.float64)) ** 2).sum())
              for i, (a, b) in enumerate(zip(xs, refs)) if i not in skip)
    den = sum(float((np.asarray(b, np.float64) ** 2).sum()) for i, b in enumerate(refs) if i not in skip)
    return (num / (den + 1e-300)) ** 0.5
