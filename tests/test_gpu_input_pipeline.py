"""The asynchronous input pipeline (pinned staging, prefetch of the next micro-batch's ids / labels / mask / document
ids, losses read late) gives the same losses, in order, and the same parameters as the blocking loop."""
import numpy as np
import pytest

from tests.golden_io import load_gpt_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["rms_swiglu_alibi_accum", "tile_docs_learned"])
def test_pipeline_equals_blocking_loop(name):
    import torch
    from tests import gpu_util
    nnb = gpu_util.nnb
    case = load_gpt_case(name)
    c, kw = case["cfg"], case["kw"]
    steps, accum = kw["steps"], kw.get("accum", 1)

    def make():
        cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, nnb.FP32)
        tr = nnb.GptTrainer(cfg, lr=kw["lr"], weight_decay=kw.get("wd", 0.01))
        tr.load_params(case["params"])
        return tr
    a = make()
    want = []
    it = iter(case["batches"])
    for _ in range(steps):
        for k in range(accum):
            mb = next(it)
            a.micro_step(mb["tokens"], mb["labels"], mb["mask"], mb["doc_ids"], grad_scale=1.0 / accum)
            want.append(float(a.loss_tensor().item()))
        a.optimizer_step(clip=kw.get("clip"))
    b = make()
    pipe = nnb.AsyncInputPipeline(b, depth=3)
    mbs = case["batches"][:steps * accum]
    sub = lambda m: pipe.submit(m["tokens"], m["labels"], m["mask"], m["doc_ids"])
    sub(mbs[0])
    j = 0
    for _ in range(steps):
        for k in range(accum):
            if j + 1 < len(mbs):
                sub(mbs[j + 1])
            pipe.run(grad_scale=1.0 / accum)
            j += 1
        b.optimizer_step(clip=kw.get("clip"))
    got = pipe.drain()
    torch.cuda.synchronize()
    assert got == want                                          # same kernels, same inputs: bit-identical
    for x, y in zip(a.get_params(), b.get_params()):
        assert np.array_equal(x, y)
    assert pipe.drain() == []
    with pytest.raises(RuntimeError):
        pipe.run()
