#!/usr/bin/env python
"""Kernel microbenchmarks through the C ABI (BASELINE configuration 5): bf16 inputs, values N(0,1) from a seed.

  python neuralnet.cpp_b200/microbench.py                   the whole sweep, one JSON line per case
  python neuralnet.cpp_b200/microbench.py --only gemm        one family: gemm | attention | ce | rmsnorm | step_gemms | linear_swiglu
  python neuralnet.cpp_b200/microbench.py --only train_step --shape 2,16 --iters 2 --no-time
                                                             training steps of a shallow copy of the benchmark model (layers,
                                                             micro-batch): every kernel of the step on ~2 GB, for profiler captures
  python neuralnet.cpp_b200/microbench.py --only decode      incremental decoding (forward_step) of the benchmark model
  python neuralnet.cpp_b200/microbench.py --only gemm --shape 16384,4096,768 --iters 3 --no-time
                                                             a few launches of one shape (for an ncu capture)

Each case is timed with CUDA events on the launching stream after 3 warm-up launches; inputs are larger than L2
or L2 is flushed between launches (--flush-l2).  `frac` is achieved / measured peak (MEASURED_PEAKS.json at the
repository root: cuBLAS bf16 burst for tensor-bound kernels, copy bandwidth for HBM-bound ones).
"""
import argparse
import ctypes as C
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

import torch  # noqa: E402

nnb = entry.load_package()
call = nnb.call


def P(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def S():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def timed(fn, iters, flush):
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if not flush:
        # back-to-back launches inside one event pair: the launch latency of all but the first is hidden, as it
        # is inside a training step
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters
    total = 0.0
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def emit(**kw):
    print(json.dumps(kw), flush=True)


def run_gemm(M, N, K, args, a_mn=0, b_mn=0, c_bf16=1, bias=False, acc=0, tag="gemm"):
    g = torch.Generator(device="cuda").manual_seed(5)
    A = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).bfloat16()
    B = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).bfloat16()
    Cm = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if c_bf16 else torch.float32)
    bv = torch.randn(N, device="cuda", generator=g) if bias else None
    fn = lambda: call("nnb200_gemm_bf16", P(A), P(B), P(Cm), M, N, K, A.shape[1], B.shape[1], N, a_mn, b_mn, c_bf16,
                      C.c_float(1.0), P(bv), None, acc, S())
    if args.no_time:
        for _ in range(args.iters):
            fn()
        torch.cuda.synchronize()
        return
    ms = timed(fn, args.iters, args.flush_l2)
    hbm, tf, src = peaks()
    ach = 2.0 * M * N * K / ms / 1e9
    emit(kernel=tag, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, us=ms * 1e3, bound="tensor", achieved=ach, peak=tf, unit="TFLOP/s",
         frac=ach / tf, peak_source=src)


def run_attention(B, S_, H, dk, args):
    g = torch.Generator(device="cuda").manual_seed(5)
    d, N = H * dk, B * S_
    qkv = torch.randn(N, 3 * d, device="cuda", generator=g).bfloat16()
    dout = torch.randn(N, d, device="cuda", generator=g).bfloat16()
    out = torch.zeros(N, d, device="cuda", dtype=torch.bfloat16)
    dqkv = torch.zeros_like(qkv)
    lse = torch.zeros(B * H * S_, device="cuda")
    dvec = torch.zeros_like(lse)
    fwd = lambda: call("nnb200_attention_forward", P(qkv), P(out), P(lse), None, None, B, S_, H, dk, 0, 1, S())
    bwd = lambda: call("nnb200_attention_backward", P(qkv), P(out), P(dout), P(lse), P(dvec), P(dqkv), None, None, B, S_, H, dk, 0, 1, S())
    if args.no_time:
        for _ in range(args.iters):
            fwd()
            bwd()
        torch.cuda.synchronize()
        return
    hbm, tf, src = peaks()
    fl = 4.0 * B * H * S_ * S_ * dk * 0.5
    for name, fn, flops in (("attention_fwd", fwd, fl), ("attention_bwd", bwd, 2.5 * fl)):
        ms = timed(fn, args.iters, args.flush_l2)
        ach = flops / ms / 1e9
        emit(kernel=name, batch=B, seq=S_, heads=H, head_dim=dk, us=ms * 1e3, bound="tensor", achieved=ach, peak=tf,
             unit="TFLOP/s", frac=ach / tf, peak_source=src)


def run_linear_swiglu(M, ff, K, args):
    """First feed-forward projection + SwiGLU: one launch (the GEMM's SwiGLU epilogue) against GEMM + activation kernel."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * ff, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = torch.randn(2 * ff, device="cuda", generator=g)
    h1 = torch.empty(M, 2 * ff, device="cuda", dtype=torch.bfloat16)
    h2 = torch.empty(M, ff, device="cuda", dtype=torch.bfloat16)
    fused = lambda: call("nnb200_linear_swiglu_forward", P(x), P(w), P(b), P(h1), P(h2), M, ff, K, S())

    def two():
        call("nnb200_gemm_bf16", P(x), P(w), P(h1), M, 2 * ff, K, K, K, 2 * ff, 0, 0, 1, C.c_float(1.0), P(b), None, 0, S())
        call("nnb200_activation_forward", P(h1), P(h2), M, ff, 1, 1, S())
    # backward: input gradient of the second projection taken through the activation (dY: (M, K), W2: (K, ff))
    w2 = (torch.randn(K, ff, device="cuda", generator=g) * 0.05).bfloat16()
    dh2 = torch.empty(M, ff, device="cuda", dtype=torch.bfloat16)
    dh1 = torch.empty(M, 2 * ff, device="cuda", dtype=torch.bfloat16)
    part = torch.empty((M + 127) // 128, 2 * ff, device="cuda")  # column sums per 128 rows, as the training step asks for them
    fused_b = lambda: call("nnb200_linear_swiglu_backward", P(x), P(w2), P(h1), P(dh1), M, ff, K, P(part), S())

    bsum = torch.zeros(2 * ff, device="cuda")
    bscratch = torch.empty(int(nnb.lib.nnb200_colsum_scratch_floats(M, 2 * ff)), device="cuda")

    def two_b():                                                   # GEMM, activation backward, bias-gradient column sums
        call("nnb200_gemm_bf16", P(x), P(w2), P(dh2), M, ff, K, K, ff, ff, 0, 1, 1, C.c_float(1.0), None, None, 0, S())
        call("nnb200_activation_backward", P(dh2), P(h1), P(dh1), M, ff, 1, 1, S())
        call("nnb200_bias_grad", P(dh1), 2 * ff, P(bsum), P(bscratch), M, 2 * ff, 1, S())
    fused()
    if args.no_time:
        for _ in range(args.iters):
            fused()
            fused_b()
        torch.cuda.synchronize()
        return
    hbm, tf, src = peaks()
    for name, fn, fl in (("linear_swiglu.fused", fused, 4.0), ("linear_swiglu.two_kernels", two, 4.0),
                         ("linear_swiglu_backward.fused", fused_b, 2.0), ("linear_swiglu_backward.two_kernels", two_b, 2.0)):
        ms = timed(fn, args.iters, args.flush_l2)
        ach = fl * M * ff * K / ms / 1e9
        emit(kernel=name, M=M, ff=ff, K=K, us=ms * 1e3, bound="tensor", achieved=ach, peak=tf, unit="TFLOP/s", frac=ach / tf,
             peak_source=src)


def run_ce(rows, V, args):
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(rows, V, device="cuda", generator=g).bfloat16()
    work = torch.empty_like(logits)
    labels = torch.randint(0, V, (rows,), device="cuda", generator=g, dtype=torch.int32)
    lv, st, lo = torch.zeros(rows, device="cuda"), torch.zeros(2, device="cuda"), torch.zeros(1, device="cuda")

    def fn():
        work.copy_(logits)          # the kernel overwrites its input; the copy is outside the timed kernel below
    fn()
    ce = lambda: call("nnb200_cross_entropy", P(work), P(labels), None, C.c_float(1.0), P(lv), P(st), P(lo), rows, V, V, 1, S())
    if args.no_time:
        for _ in range(args.iters):
            ce()
        torch.cuda.synchronize()
        return
    ms = timed(ce, args.iters, args.flush_l2)
    hbm, tf, src = peaks()
    ach = 2.0 * rows * V * 2 / ms / 1e6
    emit(kernel="cross_entropy", rows=rows, vocab=V, us=ms * 1e3, bound="hbm", achieved=ach, peak=hbm, unit="GB/s",
         frac=ach / hbm, peak_source=src)


def run_rmsnorm(rows, d, args):
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    gy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    y, dx = torch.empty_like(x), torch.empty_like(x)
    gamma, dgamma = torch.ones(d, device="cuda"), torch.zeros(d, device="cuda")
    rinv = torch.zeros(rows, device="cuda")
    scratch = torch.zeros(int(call("nnb200_colsum_scratch_floats", rows, d)), device="cuda")
    fwd = lambda: call("nnb200_norm_forward", P(x), P(gamma), None, P(y), P(rinv), None, rows, d, 0, 1, S())
    bwd = lambda: call("nnb200_norm_backward", P(gy), P(x), P(gamma), P(rinv), None, None, P(dx), P(dgamma), None, P(scratch),
                       rows, d, 0, 1, S())
    if args.no_time:
        for _ in range(args.iters):
            fwd()
            bwd()
        torch.cuda.synchronize()
        return
    hbm, tf, src = peaks()
    for name, fn, nbytes in (("rmsnorm_fwd", fwd, 2.0 * rows * d * 2 + rows * 4), ("rmsnorm_bwd", bwd, 3.0 * rows * d * 2)):
        ms = timed(fn, args.iters, args.flush_l2)
        ach = nbytes / ms / 1e6
        emit(kernel=name, rows=rows, d=d, us=ms * 1e3, bound="hbm", achieved=ach, peak=hbm, unit="GB/s", frac=ach / hbm,
             peak_source=src)


def run_decode(context, args):
    """Incremental decoding of the benchmark model (d 768, 12 layers, vocab 8192, bf16 weights): `forward_step` with
    `context` tokens already in the key / value cache.  Bound: every weight is read once per token (2 bytes each)."""
    cfg = nnb.GptConfig(8192, 768, 12, 12, 2048, 1024, 1, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_ALIBI, nnb.BF16)
    tr = nnb.GptTrainer(cfg, lr=1e-3)
    tr.init_params_normal(seed=42, std=0.02)
    for t in range(context):                       # fill the cache
        tr.forward_step(t % 8192, t, t)
    fn = lambda: tr.forward_step(17, context, context)
    if args.no_time:
        for _ in range(args.iters):
            fn()
        torch.cuda.synchronize()
        return
    hbm, tf, src = peaks()
    ms = timed(fn, args.iters, args.flush_l2)
    nbytes = 2.0 * tr.arena_elems                  # the bf16 copy of every parameter (learned positions and padding included)
    ach = nbytes / ms / 1e6
    emit(kernel="decode_forward_step", context=context, us=ms * 1e3, tokens_per_s=1e3 / ms, bound="hbm", achieved=ach, peak=hbm,
         unit="GB/s", frac=ach / hbm, peak_source=src)


def run_train_step(layers, batch, args):
    """The benchmark model (d 768, 12 heads, SwiGLU 2048, RMSNorm, ALiBi, vocab 8192, seq 1024, bf16) with `layers` layers:
    forward + loss + backward + AdamW per step, token ids from a seed."""
    cfg = nnb.GptConfig(8192, 768, 12, layers, 2048, 1024, batch, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_ALIBI, nnb.BF16)
    tr = nnb.GptTrainer(cfg, lr=3e-4, weight_decay=0.01)
    tr.init_params_normal(seed=42, std=0.02)
    g = torch.Generator(device="cuda").manual_seed(7)
    ids = torch.randint(0, 8192, (batch, 1025), device="cuda", generator=g, dtype=torch.int32)
    tok, lab = ids[:, :-1].reshape(-1).contiguous(), ids[:, 1:].reshape(-1).contiguous()
    mask = torch.ones(batch * 1024, device="cuda")

    def step():
        tr.micro_step(tok, lab, mask, None, grad_scale=1.0, last=True)
        tr.optimizer_step(lr=3e-4)
    if args.no_time:
        for _ in range(args.iters):
            step()
        torch.cuda.synchronize()
        return
    ms = timed(step, args.iters, False)
    emit(kernel="train_step", layers=layers, micro_batch=batch, seq=1024, ms=ms, tokens_per_s=batch * 1024 / ms * 1e3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="all")
    ap.add_argument("--shape", default=None, help="comma-separated override: gemm M,N,K | attention B,S,H,dk | ce rows,V | rmsnorm rows,d | linear_swiglu M,ff,K")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--no-time", action="store_true", help="just launch --iters times (for profiler captures)")
    args = ap.parse_args()
    shape = [int(v) for v in args.shape.split(",")] if args.shape else None
    fam = args.only
    if fam in ("all", "gemm"):
        for s in ([shape] if shape else [(n, n, n) for n in (1024, 2048, 4096, 8192)]):
            run_gemm(*s, args)
    if fam in ("all", "step_gemms"):
        # the GEMMs of one config-3 layer: forward (K-major x K-major), input gradient, weight gradient (split-K)
        T = 16384
        for n, k, tag in ((2304, 768, "qkv"), (768, 768, "out_proj"), (4096, 768, "fc1"), (768, 2048, "fc2"), (8192, 768, "lm_head")):
            run_gemm(T, n, k, args, bias=True, tag=tag + ".fwd")
            run_gemm(T, k, n, args, b_mn=1, tag=tag + ".dx")
            run_gemm(n, k, T, args, a_mn=1, b_mn=1, c_bf16=0, acc=1, tag=tag + ".dw")
    if fam in ("all", "linear_swiglu"):
        for s in ([shape] if shape else [(16384, 2048, 768), (8192, 2816, 1024)]):
            run_linear_swiglu(*s, args)
    if fam in ("all", "attention"):
        for s in ([shape] if shape else [(4, sq, 16, dk) for dk in (64, 128) for sq in (512, 1024, 2048, 4096, 8192)]):
            run_attention(*s, args)
    if fam in ("all", "ce"):
        run_ce(*(shape or (16384, 32768)), args)
    if fam == "train_step":
        run_train_step(*(shape or (2, 16)), args)
    if fam == "decode":
        for ctx in ([shape[0]] if shape else [16, 512, 1000]):
            run_decode(ctx, args)
    if fam in ("all", "rmsnorm"):
        run_rmsnorm(*(shape or (65536, 4096)), args)
    code = C.c_int(0)
    call("nnb200_gemm_status", C.byref(code))
    if code.value:
        raise SystemExit(f"device status word set: {code.value:#x}")


if __name__ == "__main__":
    main()
