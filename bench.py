#!/usr/bin/env python
"""Benchmark of the GPT training step (forward + backward + optimizer) on B200.

  python bench.py --gpus N --steps K --warmup W            this repository's CUDA path
  python bench.py --impl reference --gpus N --steps K ...  the reference CPU engine on the host cores
  python bench.py --config 2|4 ...                         the other training configurations (extra arms)
  python bench.py --host cpp ...                           the same step driven by the C++ host (extra arm)

Default workload: BASELINE configuration 3 — vocab 8192, d_model 768, 12 heads, 12 layers, SwiGLU FFN 2048,
RMSNorm, ALiBi, seq 1024, micro-batch 16 per GPU, gradient accumulation 2, AdamW with a cosine
schedule, fp32 master weights, bf16 tensor-core GEMM/attention; token ids Zipf(1.1) from a per-rank
seed; weights N(0, 0.02) from seed 42.  One step = one optimizer step = 2 micro-batches = 32768
tokens per GPU.  --config 2: vocab 4096, d 384, 6 heads, 6 layers, SwiGLU 1024, RMSNorm, sinusoidal, seq 256,
batch 32, AdamW 6e-4, clip 1.0.  --config 4: vocab 16384, d 1024, 16 heads, 16 layers, SwiGLU 2816, RMSNorm,
learned positions, seq 2048, batch 8 per GPU, rows packed with geometric(300) documents (attention inside a
document only), Muon on the hidden matrices + AdamW on the rest.  Prints ONE JSON line on rank 0.
"""
import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    2: dict(name="BASELINE configs[1]: small GPT on one GPU", vocab=4096, d_model=384, heads=6, layers=6, d_ff=1024, seq=256,
            batch=32, accum=1, pos="sinusoidal", clip=1.0, muon=False, docs=False, seed=2, cosine=False),
    3: dict(name="BASELINE configs[2]: GPT-small-class data-parallel training step", vocab=8192, d_model=768, heads=12,
            layers=12, d_ff=2048, seq=1024, batch=16, accum=2, pos="alibi", clip=None, muon=False, docs=False, seed=1000,
            cosine=True),
    4: dict(name="BASELINE configs[3]: packed document-masked GPT, Muon + AdamW", vocab=16384, d_model=1024, heads=16,
            layers=16, d_ff=2816, seq=2048, batch=8, accum=1, pos="learned", clip=None, muon=True, docs=True, seed=2000,
            cosine=False),
}
WORKLOAD = WORKLOADS[3]
BASE_LR, MIN_LR, WARMUP_STEPS, TOTAL_STEPS, WEIGHT_DECAY, MUON_LR = 6e-4, 6e-5, 2, 1000, 0.01, 0.02
METRIC = "gpt_train_tokens_per_sec"


def flops_per_token(w, mean_keys):
    """Algorithmic training FLOPs per token: 3 * (2*[L*(4d^2 + 3*d*ff) + d*V] + 4*d*L*mean_keys)."""
    d, ff, L, V = w["d_model"], w["d_ff"], w["layers"], w["vocab"]
    return 3.0 * (2.0 * (L * (4 * d * d + 3 * d * ff) + d * V) + 4.0 * d * L * mean_keys)


def muon_flops_per_step(w):
    """Newton-Schulz work of one Muon step on the short side: 5 * sum over hidden matrices of 4 r^2 c + 2 r^3,
    r = min(rows, cols), c = max(rows, cols)."""
    d, ff, L = w["d_model"], w["d_ff"], w["layers"]
    total = 0.0
    for rows, cols in [(d, d)] * 4 + [(2 * ff, d), (d, ff)]:
        r, c = min(rows, cols), max(rows, cols)
        total += 4.0 * r * r * c + 2.0 * r ** 3
    return 5.0 * L * total


def step_lr(step, w=None):
    """compute_step_lr of the reference (cli/lr_scheduler.hpp:89-114): linear warm-up, cosine decay."""
    if w is not None and not w["cosine"]:
        return BASE_LR
    if WARMUP_STEPS > 0 and step < WARMUP_STEPS:
        return BASE_LR * (step + 1) / WARMUP_STEPS
    p = min(max((step - WARMUP_STEPS) / max(TOTAL_STEPS - WARMUP_STEPS, 1), 0.0), 1.0)
    return MIN_LR + 0.5 * (BASE_LR - MIN_LR) * (1.0 + math.cos(math.pi * p))


def zipf_tokens(rng, vocab, n, s=1.1):
    import numpy as np
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(w) / w.sum()
    return np.minimum(np.searchsorted(cdf, rng.random(n)), vocab - 1).astype(np.int32)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(prefix="nnb200_clocks_", suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    mx.append(float(f[1]))
                except ValueError:
                    continue
                for n, v in zip(names, f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            busy = sorted(x for x in sm if x > 0.5 * max(sm)) or sorted(sm)
            out.update(sm_mhz=busy[len(busy) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CpuEngine (oracle/_ref/ref_gpt)
# --------------------------------------------------------------------------------------
POS_IDS = {"learned": 0, "sinusoidal": 1, "alibi": 2}


def run_cpu_reference(steps, cfg_id=3):
    """Times the unmodified reference CPU engine (GPTModel + CrossEntropyLoss::forward_sparse + the configuration's
    optimizers on CpuEngine, all host threads) on a bounded sample of the workload.  Configuration 3: the full model
    shape, one sequence of 1024 tokens per step (batch 1 instead of 16, no accumulation).  Configuration 2: the full
    configuration (batch 32).  Configuration 4: full width, two of the sixteen layers, one packed row of 2048 tokens
    (the reference's Newton-Schulz runs in the stored orientation: minutes per layer on host cores)."""
    import numpy as np
    from oracle import gpt_oracle as go
    from oracle import ref_runner as rr
    w = WORKLOADS[cfg_id]
    batch = {2: w["batch"], 3: 1, 4: 1}[cfg_id]
    layers = 2 if cfg_id == 4 else w["layers"]
    cfg = go.GptConfig(w["vocab"], w["d_model"], w["heads"], layers, w["d_ff"], w["seq"], batch,
                       go.ACT_SWIGLU, go.NORM_RMS, POS_IDS[w["pos"]])
    params = go.init_params(cfg, 42)
    mbs = go.make_batches(cfg, steps, seed=w["seed"], dist="zipf", docs=w["docs"])
    kw = dict(steps=steps, lr=BASE_LR, wd=WEIGHT_DECAY, skip_params=True)
    if w["cosine"]:
        kw.update(cosine=True, warmup=WARMUP_STEPS, total_steps=TOTAL_STEPS, min_lr=MIN_LR)
    if w["clip"]:
        kw.update(clip=w["clip"])
    if w["muon"]:
        kw.update(optimizer=go.OPT_MUON_SPLIT, muon_lr=MUON_LR)
    out = rr.run_reference(cfg, params, mbs, **kw)
    secs = out["seconds"]
    tokens = cfg.tokens
    what = {2: f"the full configuration (batch {batch} x {w['seq']} tokens)",
            3: f"1 sequence x {w['seq']} tokens (batch 1, no accumulation) at the full model shape",
            4: f"1 packed row x {w['seq']} tokens at full width, {layers} of {w['layers']} layers"}[cfg_id]
    return dict(value=tokens * len(secs) / float(secs.sum()), unit="tokens/s", cores=os.cpu_count(), kind="reference",
                sample=f"{len(secs)} step(s) of {what}: forward + backward + optimizer on the reference CpuEngine",
                ms_per_step=1e3 * float(secs.mean()), last_loss=float(out["losses"][-1]))


def reference_arm(args, rank):
    if rank != 0:
        return 0
    steps = max(1, min(args.steps, 3))      # about a minute of CPU work per step: bounded so the arm ends in minutes
    line = {"impl": "reference", "metric": METRIC, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": 0, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_dict(args.gpus, args.config)}
    try:
        cb = run_cpu_reference(steps, args.config)
    except Exception as e:  # the harness binary is built where the reference tree is present
        print(json.dumps({"impl": "reference", "unavailable": f"reference CPU harness not runnable: {e}"[:300]}))
        return 0
    line.update(value=cb["value"], ms_per_step=cb["ms_per_step"],
                cpu_baseline={k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                e2e={"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                gpu_launches=0)
    print(json.dumps(line))
    return 0


def config_dict(n_gpus, cfg_id=3):
    w = WORKLOADS[cfg_id]
    opt = {2: "AdamW lr 6e-4, clip 1.0, fp32 master weights", 3: "AdamW, cosine LR, fp32 master weights",
           4: "Muon (5 Newton-Schulz iterations) on the hidden matrices + AdamW on the rest, fp32 master weights"}[cfg_id]
    return {"workload": w["name"],
            "vocab": w["vocab"], "d_model": w["d_model"], "heads": w["heads"], "layers": w["layers"], "d_ff": w["d_ff"],
            "activation": "SwiGLU", "norm": "RMSNorm", "positions": {"alibi": "ALiBi"}.get(w["pos"], w["pos"]), "seq_len": w["seq"],
            "micro_batch_per_gpu": w["batch"], "grad_accum": w["accum"],
            "global_batch": w["batch"] * w["accum"] * n_gpus, "optimizer": opt,
            "documents": "rows packed with geometric(mean 300) documents, attention inside a document" if w["docs"] else "none",
            "parallelism": f"dp{n_gpus}", "l2": "working set per step (GBs of activations) exceeds the 126 MB L2"}


def packed_doc_ids(rng, batch, seq, mean_len=300.0):
    """Rows packed with documents whose lengths are geometric(mean_len), truncated at the row end; ids 1, 2, ..."""
    import numpy as np
    out = np.zeros((batch, seq), np.int32)
    for b in range(batch):
        t, d = 0, 1
        while t < seq:
            n = int(rng.geometric(1.0 / mean_len))
            out[b, t:t + n] = d
            t, d = t + n, d + 1
    return out


def mean_allowed_keys(docs, seq):
    """Mean number of keys a query may attend to: (S+1)/2 for plain causal attention, else counted from the document ids
    (position inside the document + 1, averaged)."""
    import numpy as np
    if docs is None:
        return (seq + 1) / 2.0
    d = docs.reshape(-1, seq)
    total = 0
    for row in d:
        start = np.concatenate([[0], np.nonzero(np.diff(row))[0] + 1])
        first = start[np.searchsorted(start, np.arange(seq), side="right") - 1]
        total += int((np.arange(seq) - first + 1).sum())
    return total / d.size


# --------------------------------------------------------------------------------------
# the C++ host arm: neuralnet.cpp_b200/engine/build/fused_train bench (configuration 3, one GPU)
# --------------------------------------------------------------------------------------
def cpp_host_arm(args):
    exe = os.path.join(ROOT, "neuralnet.cpp_b200", "engine", "build", "fused_train")
    if not os.path.isfile(exe):
        print(json.dumps({"host": "cpp", "unavailable": "fused_train is built where the reference headers are present "
                          "(make -C neuralnet.cpp_b200/engine REF=<reference tree>)"}))
        return 0
    r = subprocess.run([exe, "bench", "--steps", str(max(1, args.steps)), "--warmup", str(max(0, args.warmup))],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise SystemExit("fused_train bench failed: " + r.stderr[-2000:])
    cpp = json.loads(r.stdout.strip().splitlines()[-1])
    w = WORKLOADS[3]
    line = {"metric": METRIC, "value": cpp["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": cpp["steps"],
            "warmup": cpp["warmup"], "ms_per_step": cpp["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(1, 3), "host": "cpp",
            "e2e": {"value": cpp["e2e_tokens_per_s"], "unit": "tokens/s", "ms_per_step": cpp["e2e_ms_per_step"],
                    "h2d_bytes_per_step": w["accum"] * w["batch"] * w["seq"] * (4 + 4), "d2h_bytes_per_step": w["accum"] * 4,
                    "last_loss": cpp["last_loss"]},
            "gpu_launches": cpp["gpu_launches"]}
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------
# this repository's arm
# --------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", type=int, default=3, choices=[2, 3, 4], help="BASELINE training configuration (default 3, the headline)")
    ap.add_argument("--host", default="python", choices=["python", "cpp"], help="cpp: the C++ Layer/Optimizer host (configuration 3, 1 GPU)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU leg (rank 0, N=1 only)")
    ap.add_argument("--grad-buckets", default="fp32", choices=["fp32", "bf16"],
                    help="dtype the gradient buckets are all-reduced in at N > 1 (bf16: half the bytes, gradients rounded once per rank)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return reference_arm(args, rank)
    if args.host == "cpp":
        return cpp_host_arm(args) if rank == 0 else 0

    import numpy as np
    import torch
    import __graft_entry__ as entry
    nnb = entry.load_package()          # raises if libnnb200.so is missing: there is no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    pg = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
        pg = dist.group.WORLD
    w = WORKLOADS[args.config]
    K, W = max(1, args.steps), max(0, args.warmup)
    pos = {"learned": nnb.POS_LEARNED, "sinusoidal": nnb.POS_SINUSOIDAL, "alibi": nnb.POS_ALIBI}[w["pos"]]
    cfg = nnb.GptConfig(w["vocab"], w["d_model"], w["heads"], w["layers"], w["d_ff"], w["seq"], w["batch"],
                        nnb.ACT_SWIGLU, nnb.NORM_RMS, pos, nnb.BF16)
    tr = nnb.GptTrainer(cfg, lr=BASE_LR, weight_decay=WEIGHT_DECAY, muon=w["muon"], muon_lr=MUON_LR, process_group=pg,
                        grad_reduce_dtype=args.grad_buckets)
    tr.init_params_normal(seed=42, std=0.02)
    ntok, accum = w["batch"] * w["seq"], w["accum"]

    # synthetic data: per-rank seed, S+1 ids per row, x = ids[:S], y = ids[1:], mask of ones
    rng = np.random.default_rng(w["seed"] + rank)
    n_micro = accum * 4                   # a small pool of distinct micro-batches, cycled
    ids = zipf_tokens(rng, w["vocab"], n_micro * w["batch"] * (w["seq"] + 1)).reshape(n_micro, w["batch"], w["seq"] + 1)
    host_tok = torch.from_numpy(np.ascontiguousarray(ids[:, :, :-1]).reshape(n_micro, ntok)).pin_memory()
    host_lab = torch.from_numpy(np.ascontiguousarray(ids[:, :, 1:]).reshape(n_micro, ntok)).pin_memory()
    host_mask = torch.ones(n_micro, ntok, dtype=torch.float32).pin_memory()
    docs_np = np.stack([packed_doc_ids(rng, w["batch"], w["seq"]).reshape(-1) for _ in range(n_micro)]) if w["docs"] else None
    host_doc = torch.from_numpy(docs_np).pin_memory() if w["docs"] else None
    dev_tok, dev_lab, dev_mask = host_tok.cuda(), host_lab.cuda(), host_mask.cuda()
    dev_doc = host_doc.cuda() if w["docs"] else None

    # end to end: the user hands host arrays to the input pipeline (pinned staging, the copy of the next micro-batch
    # overlaps the current one, losses come back without stalling the device) — every micro-batch still crosses the
    # bus inside the timed region, and every loss is read before the region ends
    pipe = nnb.AsyncInputPipeline(tr)
    host_np = dict(tok=host_tok.numpy(), lab=host_lab.numpy(), msk=host_mask.numpy(), doc=host_doc.numpy() if w["docs"] else None)

    def submit(j):
        i = j % n_micro
        pipe.submit(host_np["tok"][i], host_np["lab"][i], host_np["msk"][i], host_np["doc"][i] if w["docs"] else None)

    def run_step(step, resident, end_step=None):
        for a in range(accum):
            j = step * accum + a
            if resident:
                i = j % n_micro
                tr.micro_step(dev_tok[i], dev_lab[i], dev_mask[i], dev_doc[i] if w["docs"] else None, grad_scale=1.0 / accum,
                              last=(a == accum - 1))
            else:
                if pipe.n_sub == pipe.n_run:
                    submit(j)                                  # the first micro-batch of a run: nothing staged yet
                if end_step is None or j + 1 < end_step * accum:
                    submit(j + 1)                              # the next one travels while this one computes
                pipe.run(grad_scale=1.0 / accum, last=(a == accum - 1))
        lr = step_lr(step, w)
        tr.optimizer_step(clip=w["clip"], lr=lr, muon_lr=lr * MUON_LR / BASE_LR)
        return None

    def timed(resident, first_step):
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for s in range(K):
            last = run_step(first_step + s, resident, first_step + K)
        if not resident:
            losses = pipe.drain()                              # every loss of the region has reached the host
            last = losses[-1] if losses else None
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
        return float(ms.item()), last

    # the sampler starts before the warm-up (nvidia-smi needs a moment before its first sample); samples taken
    # while the SMs idle are filtered out in ClockSampler.stop
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for s in range(W):
        run_step(s, True)
    torch.cuda.synchronize()
    nnb.call("nnb200_launch_count", 1)
    ms_resident, _ = timed(True, W)
    launches = int(nnb.call("nnb200_launch_count", 1))
    clocks = sampler.stop() if sampler else None
    run_step(W + K, False, W + K + 1)      # warm the host-buffer path
    pipe.drain()
    ms_e2e, last_loss = timed(False, W + K + 1)

    # roofline of the dominant kernel (tcgen05 GEMM): event pairs around every launch of one more step
    nnb.call("nnb200_gemm_profile", 1)
    tr.time_optimizer = True               # CUDA events around the Muon part of this one step
    run_step(W + 2 * K + 1, True)
    nnb.call("nnb200_gemm_profile", 0)
    tms, tfl, nl = C.c_double(0), C.c_double(0), C.c_int(0)
    nnb.call("nnb200_gemm_profile_read", C.byref(tms), C.byref(tfl), C.byref(nl))
    # the GEMM launches whose epilogue also runs the SwiGLU activation (forward: fc1, backward: fc2's input gradient)
    fms, ffl, fnl = C.c_double(0), C.c_double(0), C.c_int(0)
    nnb.call("nnb200_gemm_profile_read_fused", C.byref(fms), C.byref(ffl), C.byref(fnl))
    torch.cuda.synchronize()
    muon_ms = tr.muon_ms() if w["muon"] else None
    tr.check_device_status()

    # data-parallel cost: the same steps with the gradient all-reduce switched off (replicas drift: last measurement)
    comm = None
    if world > 1:
        tr.skip_all_reduce = True
        ms_nocomm, _ = timed(True, W + 2 * K + 2)
        tr.skip_all_reduce = False
        bytes_step = tr.arena_elems * tr.all_reduce_bytes_per_elem()
        exposed = max(ms_resident - ms_nocomm, 0.0) / K
        comm = {"all_reduce_bytes_per_step": bytes_step, "dtype": tr.grad_bucket_dtype(),
                "exposed_ms_per_step": exposed, "ms_per_step_without_all_reduce": ms_nocomm / K,
                "bus_gbs_if_exposed_only": (2.0 * (world - 1) / world) * bytes_step / (exposed * 1e-3) / 1e9 if exposed > 0 else None}

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0
    peaks = load_peaks()
    tokens_per_step = ntok * accum * world
    value = tokens_per_step * K / (ms_resident * 1e-3)
    e2e_value = tokens_per_step * K / (ms_e2e * 1e-3)
    mean_keys = mean_allowed_keys(docs_np, w["seq"])
    fpt = flops_per_token(w, mean_keys)
    step_flops = fpt * ntok * accum + (muon_flops_per_step(w) if w["muon"] else 0.0)     # per GPU
    fps = step_flops / (ms_resident / K * 1e-3)
    achieved_tf = (tfl.value / (tms.value * 1e-3)) / 1e12 if tms.value > 0 else 0.0
    peak_tf = peaks["bf16_tflops_sustained"]
    h2d = accum * ntok * (4 + 4 + 4 + (4 if w["docs"] else 0))
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_resident / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": config_dict(world, args.config),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": accum * 4,
                "last_loss": last_loss},
        "gpu_launches": launches,
        "clocks": clocks,
        "model_flops_per_token": fpt,
        "mean_allowed_keys": mean_keys,
        "mfu": {"of_nominal_2250": fps / 2.25e15, "of_measured_burst": fps / (peaks["bf16_tflops"] * 1e12),
                "of_measured_sustained": fps / (peaks["bf16_tflops_sustained"] * 1e12)},
        "roofline": {"kernel": "gemm_bf16_pair_kernel (tcgen05.mma.cta_group::2)", "bound": "tensor", "achieved": achieved_tf, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": achieved_tf / peak_tf, "traffic": None,
                     "peak_source": peaks["source"] + " cuBLAS bf16, sustained (kernel timed inside a long step)",
                     "launches_timed": nl.value, "share_of_step": tms.value / (ms_resident / K) if ms_resident else None},
    }
    if fnl.value:
        # not in `achieved`: these launches also do the work of the activation kernels they replace, and their epilogue
        # outlasts the main loop; with them the GEMM family's rate is `all_gemm_launches_tflops`
        line["roofline"]["with_activation_epilogue"] = {
            "launches": fnl.value, "ms_per_step": fms.value,
            "tflops": (ffl.value / (fms.value * 1e-3)) / 1e12 if fms.value > 0 else None,
            "all_gemm_launches_tflops": ((tfl.value + ffl.value) / ((tms.value + fms.value) * 1e-3)) / 1e12,
            "share_of_step": fms.value / (ms_resident / K) if ms_resident else None}
    if w["muon"]:
        mf = muon_flops_per_step(w)
        line["muon"] = {"ms_per_step": muon_ms, "newton_schulz_flops_per_step": mf,
                        "tflops": mf / (muon_ms * 1e-3) / 1e12 if muon_ms else None,
                        "note": "Newton-Schulz on the short side of each matrix; included in the step time and in mfu"}
    if comm:
        line["comm"] = comm
    if world == 1 and not args.no_cpu_baseline:
        try:
            cb = run_cpu_reference(1, args.config)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "reference",
                                    "sample": f"not run: {e}"[:200]}
    print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
