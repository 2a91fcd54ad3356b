"""Host-side driver of the fused GPT training step (the call a user makes).

Mirrors the training-loop order of the reference driver (src/text_train.cpp:1107-1334): per
micro-batch forward -> CrossEntropyLoss.forward_sparse -> backward with the logit gradient scaled
by 1/accum; per optimizer step an optional global-norm clip, the optimizer update and zero_grad.
PyTorch is used for device memory, streams and torch.distributed only; every computation is a call
into libnnb200.so.

Data parallelism: one process per GPU, identical replicas, each rank runs its own micro-batches;
the gradient arena is summed over ranks with NCCL all-reduces issued on a side stream, per layer
bucket, as soon as the backward pass has recorded that bucket's event; 1/world is folded into the
optimizer's gradient scale.
"""
import ctypes as C
import dataclasses
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib, checkpoint
from ._lib import GptConfigC, call

ACT_GELU, ACT_SWIGLU = 0, 1
NORM_LAYER, NORM_RMS = 0, 1
POS_LEARNED, POS_SINUSOIDAL, POS_ALIBI, POS_ROPE = 0, 1, 2, 3
FP32, BF16 = 0, 1


@dataclasses.dataclass
class GptConfig:
    """nn::GptConfig (include/neuralnet.cpp/domain_gpt.hpp:29-39) plus batch and precision."""
    vocab: int
    d_model: int
    heads: int
    layers: int
    d_ff: int
    seq: int
    batch: int
    act: int = ACT_GELU
    norm: int = NORM_LAYER
    pos: int = POS_LEARNED
    precision: int = FP32

    def c_struct(self) -> GptConfigC:
        return GptConfigC(vocab=self.vocab, d_model=self.d_model, heads=self.heads, layers=self.layers,
                          d_ff=self.d_ff, seq=self.seq, batch=self.batch, act=self.act, norm=self.norm,
                          pos=self.pos, precision=self.precision)


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def gradient_buckets(layer_begin: Sequence[int], matrix_begin: int, lm_head: Optional[Sequence[int]] = None):
    """All-reduce buckets of the gradient arena as (event index, start, end) with element ranges, in issue order.
    The LM head's weight gradient comes first: it is final after the first GEMM of the backward pass (event
    layers+1).  Then the hidden matrices of the last layer (event layers-1: the backward pass finishes them first)
    down to layer 0, then what is final only when the embedding scatter-add and the deferred bias / scale folds have
    run (event layers): the vectors-and-embeddings region around the LM head's weight.  `layer_begin` has layers+1
    entries (nnb200_gpt_layer_matrix_begin); `lm_head` = (start, end) of lm_head.W inside [0, matrix_begin), or None
    to leave it in the last bucket.  The buckets tile [0, layer_begin[-1]) exactly."""
    n = len(layer_begin) - 1
    out = []
    if lm_head is not None and lm_head[1] > lm_head[0]:
        out.append((n + 1, lm_head[0], lm_head[1]))
    out += [(l, layer_begin[l], layer_begin[l + 1]) for l in range(n - 1, -1, -1)]
    if lm_head is not None and lm_head[1] > lm_head[0]:
        if lm_head[0] > 0:
            out.append((n, 0, lm_head[0]))
        if lm_head[1] < matrix_begin:
            out.append((n, lm_head[1], matrix_begin))
    else:
        out.append((n, 0, matrix_begin))
    return out


class GptTrainer:
    """Owns the parameter/gradient/moment arenas and the activation workspace of one replica."""

    def __init__(self, cfg: GptConfig, device: Optional[torch.device] = None, *, lr=1e-3, weight_decay=0.01,
                 beta1=0.9, beta2=0.999, eps=1e-8, muon: bool = False, muon_lr=0.02, muon_momentum=0.95,
                 ns_steps=5, ns_eps=1e-7, process_group=None, grad_reduce_dtype: str = "fp32"):
        if not torch.cuda.is_available():
            raise RuntimeError("GptTrainer needs a CUDA device: there is no CPU path")
        self.cfg = cfg
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self._c = cfg.c_struct()
        cp = C.byref(self._c)
        n = call("nnb200_gpt_param_table", cp, None, None, None)
        offs, rows, cols = (C.c_longlong * n)(), (C.c_int32 * n)(), (C.c_int32 * n)()
        call("nnb200_gpt_param_table", cp, offs, rows, cols)
        self.table = [(int(offs[i]), int(rows[i]), int(cols[i])) for i in range(n)]
        self.arena_elems = int(call("nnb200_gpt_arena_elems", cp))
        self.matrix_begin = int(call("nnb200_gpt_matrix_region_begin", cp))
        self.layer_begin = [int(call("nnb200_gpt_layer_matrix_begin", cp, l)) for l in range(cfg.layers + 1)]
        f32 = dict(dtype=torch.float32, device=self.device)
        self.params = torch.zeros(self.arena_elems, **f32)
        self.grads = torch.zeros(self.arena_elems, **f32)
        self.m = torch.zeros(self.arena_elems, **f32)
        self.v = torch.zeros(self.arena_elems, **f32)
        self.shadow = (torch.zeros(self.arena_elems, dtype=torch.bfloat16, device=self.device)
                       if cfg.precision == BF16 else None)
        self.ws_bytes = int(call("nnb200_gpt_workspace_bytes", cp))
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=self.device)
        call("nnb200_gpt_init_workspace", cp, _ptr(self.workspace), _stream())
        self._off = {k: int(call("nnb200_gpt_workspace_offset", cp, i))
                     for i, k in enumerate(("logits", "loss", "grad_x0", "ce_stats"))}
        self.scal = torch.zeros(8, **f32)                                  # [0..2] clip outputs
        self.sumsq_scratch = torch.empty(int(call("nnb200_sumsq_scratch_floats")), **f32)
        self.lr, self.wd, self.b1, self.b2, self.eps = lr, weight_decay, beta1, beta2, eps
        self.t = 0
        self.muon = muon
        self.muon_lr, self.muon_mu, self.ns_steps, self.ns_eps = muon_lr, muon_momentum, ns_steps, ns_eps
        if muon:
            # the hidden matrices as host arrays of device pointers for nnb200_muon_step_many; the Newton-Schulz GEMMs of
            # one matrix fill a fraction of the machine, so the matrices go round-robin over several streams ("lanes")
            mats = [(o, r, c) for o, r, c in self.table if o >= self.matrix_begin]
            worst = max(int(call("nnb200_muon_scratch_bytes", r, c, cfg.precision)) for _, r, c in mats)
            self.muon_lane_bytes = (worst + 255) // 256 * 256
            self.muon_lanes = max(1, min(8, len(mats)))
            self.muon_scratch = torch.empty(self.muon_lane_bytes * self.muon_lanes, dtype=torch.uint8, device=self.device)
            n = len(mats)
            PA, IA = C.c_void_p * n, C.c_int * n
            base = lambda t, esz: [t.data_ptr() + esz * o for o, _, _ in mats]
            self._muon_args = (n, PA(*base(self.params, 4)), PA(*base(self.grads, 4)), PA(*base(self.m, 4)),
                               PA(*base(self.shadow, 2)) if self.shadow is not None else None,
                               IA(*[r for _, r, _ in mats]), IA(*[c for _, _, c in mats]))
        # data parallel state
        self.pg = process_group
        self.world = torch.distributed.get_world_size(process_group) if process_group is not None else 1
        self.side = torch.cuda.Stream(device=self.device) if self.world > 1 else None
        self.events = [torch.cuda.Event() for _ in range(cfg.layers + 2)]
        self._event_handles = (C.c_void_p * (cfg.layers + 2))()
        lm_off, lm_r, lm_c = self.table[-2]                                 # lm_head.W
        self.buckets = gradient_buckets(self.layer_begin, self.matrix_begin, (lm_off, lm_off + lm_r * lm_c))
        # gradient buckets cross NVLink as fp32 (bit-for-bit the sum NCCL forms) or, halving the bytes and the time
        # NCCL's kernels hold SMs, as bf16 (converted on the side stream; only with the bf16 compute path)
        if grad_reduce_dtype not in ("fp32", "bf16"):
            raise ValueError("grad_reduce_dtype is 'fp32' or 'bf16'")
        self.grad_reduce_dtype = grad_reduce_dtype
        self._bf16_stage = (torch.empty(max(hi - lo for _, lo, hi in self.buckets), dtype=torch.bfloat16, device=self.device)
                            if (self.world > 1 and grad_reduce_dtype == "bf16") else None)
        self.skip_all_reduce = False          # benchmark switch: measures the step without its exchange
        self.time_optimizer = False           # CUDA events around the Muon part of the next optimizer_step
        self._muon_events = None
        self.launches = 0

    # -------------------------------------------------------------- parameters
    def load_params(self, tensors: Sequence[np.ndarray]):
        """Copies parameters given in the reference order (GPTModel::parameters) into the arena —
        the analogue of engine.copy_from(param, Matrix) on every parameter."""
        assert len(tensors) == len(self.table)
        host = np.zeros(self.arena_elems, np.float32)
        for (off, r, c), t in zip(self.table, tensors):
            host[off:off + r * c] = np.asarray(t, np.float32).reshape(-1)
        self.params.copy_(torch.from_numpy(host))
        self.refresh_shadow()

    def param_names(self) -> List[str]:
        """Names of the tensors in the reference's parameter order (GPTModel::parameters,
        compute_layer.hpp:2739-2755; GPTBlock :2336-2346)."""
        c = self.cfg
        norm = lambda p: [p + ".gamma"] + ([p + ".beta"] if c.norm == NORM_LAYER else [])
        names = ["token_emb"] + (["pos_emb"] if c.pos == POS_LEARNED else [])
        for l in range(c.layers):
            p = f"blk{l}."
            for w in ("wq", "wk", "wv", "wo"):
                names += [p + w + ".W", p + w + ".b"]
            names += norm(p + "norm1") + [p + "fc1.W", p + "fc1.b", p + "fc2.W", p + "fc2.b"] + norm(p + "norm2")
        names += norm("ln_f") + ["lm_head.W", "lm_head.b"]
        assert len(names) == len(self.table)
        return names

    def init_params_normal(self, seed=42, std=0.02):
        """Synthetic weights: matrices and embeddings ~ N(0, std), biases 0, norm scales 1 — the same
        on every rank for the same seed."""
        rng = np.random.default_rng(seed)
        tensors = []
        for name, (_, r, c) in zip(self.param_names(), self.table):
            if name.endswith(".gamma"):
                tensors.append(np.ones((r, c), np.float32))
            elif c == 1:
                tensors.append(np.zeros((r, c), np.float32))
            else:
                tensors.append((rng.standard_normal((r, c)) * std).astype(np.float32))
        self.load_params(tensors)

    def refresh_shadow(self):
        if self.shadow is not None:
            call("nnb200_f32_to_bf16", _ptr(self.params), _ptr(self.shadow), self.arena_elems, _stream())

    def _split(self, arena: torch.Tensor) -> List[np.ndarray]:
        host = arena.detach().cpu().numpy()
        return [host[off:off + r * c].reshape(r, c).copy() for off, r, c in self.table]

    def get_params(self) -> List[np.ndarray]:
        return self._split(self.params)

    def get_grads(self) -> List[np.ndarray]:
        return self._split(self.grads)

    # -------------------------------------------------------------- checkpoints
    def load_reference_checkpoint(self, path: str) -> bytes:
        """Loads the parameters of a model file written by the reference (save_model, format v4,
        model_serialization.hpp:389-428) — the analogue of load_model: the stored model description must match
        this trainer's configuration and every matrix the shape the model expects.  Returns the embedded
        tokenizer JSON (empty if none)."""
        spec, buf, off = checkpoint.read_model_file(path)
        checkpoint.check_spec_against_config(spec, self.cfg)
        mats, tok = checkpoint.split_matrices(buf, off, [(r, c) for _, r, c in self.table])
        self.load_params(mats)
        return tok

    def save_reference_checkpoint(self, path: str, tokenizer: bytes = b""):
        """Writes the fp32 master weights as a reference model file that load_model / text_train --resume /
        text_infer read."""
        checkpoint.write_model_file(path, checkpoint.spec_of_config(self.cfg), self.get_params(), tokenizer)

    def save_training_state(self, path: str):
        """Everything a resumed run needs and the reference file lacks: parameters, Adam moments (the Muon
        velocity of the hidden matrices lives in the first-moment arena) and the step counter."""
        c = self.cfg
        host = lambda t: t.detach().cpu().numpy()
        checkpoint.save_training_state(path, {"params": host(self.params), "m": host(self.m), "v": host(self.v)}, self.t,
                                       [c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.act, c.norm, c.pos, int(self.muon)])

    def load_training_state(self, path: str):
        arenas, step, cfgv = checkpoint.load_training_state(path)
        c = self.cfg
        if cfgv != [c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.act, c.norm, c.pos, int(self.muon)]:
            raise ValueError("training state was written for a different model configuration or optimizer split")
        for name, dst in (("params", self.params), ("m", self.m), ("v", self.v)):
            if arenas[name].size != self.arena_elems:
                raise ValueError(f"training state arena '{name}' has the wrong size")
            dst.copy_(torch.from_numpy(arenas[name]))
        self.t = step
        self.grads.zero_()
        self.refresh_shadow()

    # -------------------------------------------------------------- step pieces
    def _ints(self, a):
        if isinstance(a, torch.Tensor):
            return a.to(device=self.device, dtype=torch.int32, non_blocking=True)
        return torch.from_numpy(np.ascontiguousarray(a, np.int32)).to(self.device, non_blocking=True)

    def forward(self, tokens, doc_ids=None):
        self._tokens = self._ints(tokens)
        self._docs = self._ints(doc_ids) if doc_ids is not None else None
        call("nnb200_gpt_forward", C.byref(self._c), _ptr(self.params), _ptr(self.shadow), _ptr(self.workspace),
             _ptr(self._tokens), _ptr(self._docs), _stream())

    def loss_and_grad(self, labels, mask=None, grad_scale=1.0):
        self._labels = self._ints(labels)
        if mask is not None and not isinstance(mask, torch.Tensor):
            mask = torch.from_numpy(np.ascontiguousarray(mask, np.float32)).to(self.device, non_blocking=True)
        self._mask = mask
        call("nnb200_gpt_loss", C.byref(self._c), _ptr(self.workspace), _ptr(self._labels), _ptr(self._mask),
             C.c_float(grad_scale), _stream())

    def backward(self, record_events=False):
        ev = None
        if record_events:
            for i, e in enumerate(self.events):
                e.record()            # materialises the underlying cudaEvent_t
                self._event_handles[i] = e.cuda_event
            ev = self._event_handles
        call("nnb200_gpt_backward", C.byref(self._c), _ptr(self.params), _ptr(self.shadow), _ptr(self.grads),
             _ptr(self.workspace), _ptr(self._tokens), _ptr(self._docs), ev, _stream())

    def evaluate(self, batches) -> float:
        """Evaluation pass of the reference driver (src/text_train.cpp:1367-1466): forward and sparse cross-entropy
        without backward, over an iterable of (tokens, labels[, loss_mask[, doc_ids]]); returns the per-batch losses
        averaged with each batch's count of valid targets as weight, which is what the driver prints as test_loss.
        Gradients are left untouched."""
        weighted, valid = 0.0, 0.0
        o = self._off["ce_stats"]
        for b in batches:
            tokens, labels = b[0], b[1]
            mask = b[2] if len(b) > 2 else None
            docs = b[3] if len(b) > 3 else None
            self.forward(tokens, docs)
            self.loss_and_grad(labels, mask, 1.0)          # overwrites the logits in the workspace; no gradient leaves it
            n = float(self.workspace[o:o + 4].view(torch.float32).item())     # valid targets of this batch
            weighted += float(self.loss_tensor().item()) * n
            valid += n
        return weighted / valid if valid > 0 else 0.0

    # -------------------------------------------------------------- inference with a key/value cache
    def _decode_state(self):
        if getattr(self, "_decode_ws", None) is None:
            n = int(call("nnb200_gpt_decode_workspace_bytes", C.byref(self._c)))
            self._decode_ws = torch.empty(n, dtype=torch.uint8, device=self.device)
            call("nnb200_gpt_decode_init", C.byref(self._c), _ptr(self._decode_ws), _stream())
            self._decode_logits = torch.empty(self.cfg.vocab, dtype=torch.float32, device=self.device)
        return self._decode_ws, self._decode_logits

    def forward_step(self, token_id: int, pos: int, cur_len: int, graph: bool = True) -> torch.Tensor:
        """One token through the model with the key/value cache (GPTModel::forward_step, compute_layer.hpp:2906-2950):
        writes the token's keys and values at cache row cur_len, attends over rows [0, cur_len] and returns the
        (vocab,) fp32 logits (a device tensor that the next call overwrites).

        A token is about sixty small launches, which the host cannot issue as fast as the GPU runs them.  With `graph`
        the launches are captured once as a CUDA graph (nnb200_gpt_forward_step_dev reads the token id, the position
        and the cache length from device memory, so they are the same for every token) and replayed per token after a
        one-thread kernel has written the three integers."""
        ws, logits = self._decode_state()
        if not (0 <= int(cur_len) < self.cfg.seq and 0 <= int(pos) < self.cfg.seq):
            raise ValueError("pos and cur_len must be in [0, seq)")
        if not graph:
            call("nnb200_gpt_forward_step", C.byref(self._c), _ptr(self.params), _ptr(self.shadow), _ptr(ws), int(token_id), int(pos),
                 int(cur_len), _ptr(logits), _stream())
            return logits
        if getattr(self, "_decode_graph", None) is None:
            self._step_dev = torch.zeros(4, dtype=torch.int32, device=self.device)
            args = (C.byref(self._c), _ptr(self.params), _ptr(self.shadow), _ptr(ws), _ptr(self._step_dev), _ptr(logits))
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                      # one plain run first: per-device launch attributes are set there
                call("nnb200_gpt_forward_step_dev", *args, _stream())
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                call("nnb200_gpt_forward_step_dev", *args, _stream())
            self._decode_graph = g
        call("nnb200_gpt_decode_set_step", _ptr(self._step_dev), int(token_id), int(pos), int(cur_len), _stream())
        self._decode_graph.replay()
        return logits

    def generate(self, prompt: Sequence[int], max_new_tokens: int, temperature: float = 1.0, eos_token_id: int = -1,
                 min_new_tokens: int = 0, rng: Optional[np.random.Generator] = None) -> List[int]:
        """GPTModel::generate (compute_layer.hpp:2952-3096): fills the cache with the prompt (its last seq tokens), then per
        new token softmax-samples the last logits at `temperature` (0 = arg max, first maximum wins), stops at
        eos_token_id once min_new_tokens were produced, and when the cache is full rebuilds it from the last seq-1
        tokens of the context.  Sampling is on the host, as in the reference; `rng` makes it repeatable."""
        rng = rng or np.random.default_rng()
        seq = self.cfg.seq
        context, generated = list(int(t) for t in prompt), []
        cur_len, last = 0, None

        def fill(start):
            nonlocal cur_len, last
            for t in context[start:]:
                last = self.forward_step(t, cur_len, cur_len)
                cur_len += 1
        fill(max(0, len(context) - seq))
        for step in range(max_new_tokens):
            if cur_len >= seq:                       # sliding window: keep the last seq-1 tokens
                cur_len = 0
                fill(max(0, len(context) - (seq - 1)))
            if last is None:
                raise ValueError("generate needs a non-empty prompt")
            logits = last.detach().cpu().numpy().astype(np.float32)
            if temperature > 0.0 and temperature != 1.0:
                logits = logits / np.float32(temperature)
            p = np.exp(logits - logits.max())
            p /= p.sum(dtype=np.float32)
            if temperature > 0.0:
                r, nxt = np.float32(rng.random()), self.cfg.vocab - 1
                c = np.cumsum(p, dtype=np.float32)
                hit = np.nonzero(r <= c)[0]
                if hit.size:
                    nxt = int(hit[0])
            else:
                nxt = int(np.argmax(p))
            context.append(nxt)
            if step >= min_new_tokens and nxt == eos_token_id:
                break
            generated.append(nxt)
            last = self.forward_step(nxt, cur_len, cur_len)
            cur_len += 1
        return generated

    def loss_tensor(self) -> torch.Tensor:
        """Device view of the scalar loss of the last loss_and_grad call."""
        o = self._off["loss"]
        return self.workspace[o:o + 4].view(torch.float32)

    def logits(self) -> torch.Tensor:
        """(tokens, vocab) view of the logits (their gradient after loss_and_grad)."""
        c = self.cfg
        n = c.batch * c.seq * c.vocab
        o = self._off["logits"]
        dt = torch.bfloat16 if c.precision == BF16 else torch.float32
        return self.workspace[o:o + n * dt.itemsize].view(dt).view(c.batch * c.seq, c.vocab)

    def micro_step(self, tokens, labels, mask=None, doc_ids=None, grad_scale=1.0, last=True):
        """forward + loss + backward of one micro-batch; gradients accumulate."""
        self.forward(tokens, doc_ids)
        self.loss_and_grad(labels, mask, grad_scale)
        self.backward(record_events=last and self.world > 1)
        if last and self.world > 1:
            self._all_reduce_buckets()

    # -------------------------------------------------------------- data parallel
    def _all_reduce_buckets(self):
        """Sum-all-reduce of the gradient arena in the buckets of gradient_buckets (LM head weight, one bucket per
        layer's matrices in the order the backward pass completes them, then embeddings and vectors), issued on the
        side stream behind the events the backward pass recorded."""
        import torch.distributed as dist
        if self.skip_all_reduce:
            return
        with torch.cuda.stream(self.side):
            for ev, lo, hi in self.buckets:
                self.side.wait_event(self.events[ev])
                if self._bf16_stage is None:
                    dist.all_reduce(self.grads[lo:hi], group=self.pg)
                else:
                    st = self._bf16_stage[:hi - lo]
                    s = C.c_void_p(self.side.cuda_stream)
                    call("nnb200_f32_to_bf16", C.c_void_p(self.grads.data_ptr() + 4 * lo), _ptr(st), hi - lo, s)
                    dist.all_reduce(st, group=self.pg)
                    call("nnb200_bf16_to_f32", _ptr(st), C.c_void_p(self.grads.data_ptr() + 4 * lo), hi - lo, s)
        torch.cuda.current_stream().wait_stream(self.side)

    def all_reduce_bytes_per_elem(self) -> int:
        return 2 if self.grad_reduce_dtype == "bf16" else 4

    def grad_bucket_dtype(self) -> str:
        return self.grad_reduce_dtype

    def muon_ms(self) -> Optional[float]:
        """Device time of the Muon part of the last optimizer_step that ran with time_optimizer set (synchronises)."""
        if self._muon_events is None:
            return None
        e0, e1 = self._muon_events
        e1.synchronize()
        return float(e0.elapsed_time(e1))

    # -------------------------------------------------------------- optimizer
    def optimizer_step(self, clip: Optional[float] = None, lr: Optional[float] = None,
                       muon_lr: Optional[float] = None):
        """clip_grad_norm (optional) + AdamW (+ Muon on the hidden matrices) + zero_grad.
        Optimizer::clip_grad_norm / AdamW::step / Muon::step (compute_optimizer.hpp:90-140,
        388-412, 517-590).  The clip factor and 1/world stay on the device: no host sync."""
        lr = self.lr if lr is None else lr
        s = _stream()
        pre = 1.0 / self.world
        gscale = None
        if clip is not None or self.world > 1:
            call("nnb200_grad_norm_clip", _ptr(self.grads), self.arena_elems, C.c_float(pre),
                 C.c_float(clip if clip is not None else 0.0), _ptr(self.sumsq_scratch), _ptr(self.scal), s)
            gscale = C.c_void_p(self.scal.data_ptr() + 8)
        self.t += 1
        n_adam = self.matrix_begin if self.muon else self.arena_elems
        call("nnb200_adamw_step", _ptr(self.params), _ptr(self.grads), _ptr(self.m), _ptr(self.v), _ptr(self.shadow),
             n_adam, C.c_float(lr), C.c_float(self.b1), C.c_float(self.b2), C.c_float(self.eps), C.c_float(self.wd),
             self.t, gscale, s)
        if self.muon:
            if self.time_optimizer:
                self._muon_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                self._muon_events[0].record()
            mlr = self.muon_lr if muon_lr is None else muon_lr
            n, pp, gg, vv, sh, rr_, cc_ = self._muon_args
            call("nnb200_muon_step_many", n, pp, gg, vv, sh, rr_, cc_, C.c_float(mlr), C.c_float(self.muon_mu), self.ns_steps,
                 C.c_float(self.ns_eps), self.cfg.precision, _ptr(self.muon_scratch), self.muon_lane_bytes, self.muon_lanes,
                 gscale, s)
            if self.time_optimizer:
                self._muon_events[1].record()
                self.time_optimizer = False
        call("nnb200_zero_f32", _ptr(self.grads), self.arena_elems, s)       # zero_grad

    def grad_norm(self) -> float:
        """Norm computed by the last optimizer_step that clipped (host read; synchronises)."""
        return float(self.scal[1].item())

    def check_device_status(self):
        """Raises if a bounded wait inside the tcgen05 GEMM ever gave up."""
        code = C.c_int(0)
        call("nnb200_gemm_status", C.byref(code))
        if code.value:
            raise _lib.NnbError(f"tcgen05 GEMM reported a timed-out wait (code {code.value >> 16}, block {code.value & 0xffff})")


class AsyncInputPipeline:
    """Keeps the host side of the training loop off the critical path.

    The reference loop uploads the ids, labels and loss mask of a micro-batch right before it needs them and downloads
    the scalar loss right after (CrossEntropyLoss::forward_sparse, compute_loss.hpp:259-307; src/text_train.cpp:1137-1181),
    stalling the device twice per micro-batch.  Here every micro-batch is staged in pinned host memory, copied to the
    device on a copy stream while the previous micro-batch computes, and its loss is copied back without blocking: the
    value is read `depth - 1` submissions later, when its copy has long finished.

        pipe = AsyncInputPipeline(trainer)
        for tokens, labels in data:
            pipe.submit(tokens, labels)                  # host arrays; returns at once
            ...
            pipe.run(grad_scale=1/accum, last=...)       # forward + loss + backward of the oldest staged micro-batch
        losses = pipe.drain()                            # every loss, in submission order
    """

    def __init__(self, trainer: GptTrainer, depth: int = 3):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one micro-batch computing, one being staged)")
        self.tr = trainer
        n = trainer.cfg.batch * trainer.cfg.seq
        dev = trainer.device
        self.depth = depth
        pin = lambda dt: torch.empty(n, dtype=dt).pin_memory()
        self.h_tok = [pin(torch.int32) for _ in range(depth)]
        self.h_lab = [pin(torch.int32) for _ in range(depth)]
        self.h_msk = [pin(torch.float32) for _ in range(depth)]
        self.h_doc = [pin(torch.int32) for _ in range(depth)]
        mk = lambda dt: torch.empty(n, dtype=dt, device=dev)
        self.d_tok = [mk(torch.int32) for _ in range(depth)]
        self.d_lab = [mk(torch.int32) for _ in range(depth)]
        self.d_msk = [mk(torch.float32) for _ in range(depth)]
        self.d_doc = [mk(torch.int32) for _ in range(depth)]
        self.flags = [(False, False)] * depth                   # (has mask, has document ids) per slot
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.staged = [torch.cuda.Event() for _ in range(depth)]     # H2D of the slot finished
        self.consumed = [torch.cuda.Event() for _ in range(depth)]   # the step that read the slot finished
        self.loss_host = torch.zeros(depth, dtype=torch.float32).pin_memory()
        self.loss_ready = [torch.cuda.Event() for _ in range(depth)]
        self.n_sub = self.n_run = self.n_read = 0
        self._losses: List[float] = []
        self.h2d_bytes = 0

    def submit(self, tokens, labels, mask=None, doc_ids=None):
        """Stages one micro-batch (host arrays or tensors) and starts its copy to the device."""
        if self.n_sub - self.n_run >= self.depth - 1:
            raise RuntimeError("pipeline full: call run() before submitting more")
        s = self.n_sub % self.depth
        if self.n_sub >= self.depth:
            self.consumed[s].synchronize()                     # the step that used this slot has read its buffers
        as_t = lambda a, dt: a.to(dt) if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a, {torch.int32: np.int32, torch.float32: np.float32}[dt]))
        self.h_tok[s].copy_(as_t(tokens, torch.int32).reshape(-1))
        self.h_lab[s].copy_(as_t(labels, torch.int32).reshape(-1))
        if mask is not None:
            self.h_msk[s].copy_(as_t(mask, torch.float32).reshape(-1))
        if doc_ids is not None:
            self.h_doc[s].copy_(as_t(doc_ids, torch.int32).reshape(-1))
        self.flags[s] = (mask is not None, doc_ids is not None)
        with torch.cuda.stream(self.copy_stream):
            self.d_tok[s].copy_(self.h_tok[s], non_blocking=True)
            self.d_lab[s].copy_(self.h_lab[s], non_blocking=True)
            nbytes = 8 * self.h_tok[s].numel()
            if mask is not None:
                self.d_msk[s].copy_(self.h_msk[s], non_blocking=True)
                nbytes += 4 * self.h_tok[s].numel()
            if doc_ids is not None:
                self.d_doc[s].copy_(self.h_doc[s], non_blocking=True)
                nbytes += 4 * self.h_tok[s].numel()
            self.staged[s].record(self.copy_stream)
        self.h2d_bytes += nbytes
        self.n_sub += 1

    def run(self, grad_scale: float = 1.0, last: bool = True):
        """forward + loss + backward of the oldest staged micro-batch; its loss starts its way back to the host."""
        if self.n_run >= self.n_sub:
            raise RuntimeError("nothing staged")
        s = self.n_run % self.depth
        cur = torch.cuda.current_stream()
        cur.wait_event(self.staged[s])
        has_mask, has_doc = self.flags[s]
        self._collect(self.n_run - (self.depth - 1))           # the slot's previous loss, copied long ago
        self.tr.micro_step(self.d_tok[s], self.d_lab[s], self.d_msk[s] if has_mask else None,
                           self.d_doc[s] if has_doc else None, grad_scale=grad_scale, last=last)
        self.loss_host[s:s + 1].copy_(self.tr.loss_tensor(), non_blocking=True)
        self.loss_ready[s].record(cur)
        self.consumed[s].record(cur)
        self.n_run += 1

    def _collect(self, upto: int):
        while self.n_read <= upto and self.n_read < self.n_run:
            s = self.n_read % self.depth
            self.loss_ready[s].synchronize()
            self._losses.append(float(self.loss_host[s]))
            self.n_read += 1

    def drain(self) -> List[float]:
        """Waits for every micro-batch run so far and returns all losses not handed out yet, in order."""
        self._collect(self.n_run - 1)
        out, self._losses = self._losses, []
        return out
