#!/usr/bin/env python
"""Generates tests/golden/text_train/: the inputs and reference results for running the reference's own
training driver (src/text_train.cpp, compiled unchanged into oracle/_ref/engine/text_train) on this
repository's drop-in CUDA engine.

  corpus.txt     seeded synthetic text: 120 blank-line separated "documents" of made-up words
  vocab.json     byte-level BPE vocabulary trained on it by the reference's tokenizer_train
  start.bin      a model checkpoint (the reference's v4 format) after one epoch on the reference CPU engine
  expected.json  what the reference CPU engine reports when it resumes from start.bin:
                   eval_loss   test loss with lr = 0 (deterministic: the weights never move)
                   train_loss  epoch-average training loss at lr 1e-3 over three runs (the driver shuffles
                               with std::random_device, so the value moves a little from run to run)

Needs the reference sources (the binaries are built by `make -C oracle`); run from the repository root:
    python tests/golden/make_text_train_fixture.py
"""
import json
import os
import random
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BIN = os.path.join(ROOT, "oracle", "_ref", "engine")
OUT = os.path.join(ROOT, "tests", "golden", "text_train")

MODEL_ARGS = ["--batch-size", "8", "--seq-len", "32", "--d-model", "64", "--num-heads", "4", "--num-layers", "2", "--d-ff", "128",
              "--optimizer", "adamw", "--log-interval", "50", "--no-cache", "--activation", "swiglu", "--norm", "rmsnorm",
              "--positional-encoding", "alibi", "--epochs", "1"]


def synthetic_corpus(seed=11):
    r = random.Random(seed)
    syllables = ["ka", "lo", "mi", "ten", "sur", "ba", "ri", "no", "vel", "dax", "pu", "shi", "ong", "tre", "qua", "zel", "fi", "mar"]
    words = ["".join(r.choice(syllables) for _ in range(r.randint(1, 3))) for _ in range(300)]
    docs = []
    for _ in range(120):
        sentences = []
        for _ in range(r.randint(3, 9)):
            n = r.randint(4, 12)
            s = " ".join(r.choice(words[:60]) if r.random() < 0.7 else r.choice(words) for _ in range(n))
            sentences.append(s.capitalize() + ".")
        docs.append(" ".join(sentences))
    return "\n\n".join(docs) + "\n"


def run_driver(extra, cwd):
    """Runs the reference driver; returns (epoch-average loss, test loss or None)."""
    cmd = [os.path.join(BIN, "text_train"), "corpus.txt", "--vocab", "vocab.json"] + MODEL_ARGS + extra
    out = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True, check=True).stdout.replace("\r", "\n")
    avg = re.findall(r"avg_loss=([0-9.]+)", out)
    test = re.findall(r"test_loss=([0-9.]+)", out)
    return float(avg[-1]), (float(test[-1]) if test else None)


def main():
    os.makedirs(OUT, exist_ok=True)
    with open(os.path.join(OUT, "corpus.txt"), "w") as f:
        f.write(synthetic_corpus())
    subprocess.run([os.path.join(BIN, "tokenizer_train"), "corpus.txt", "--output", "vocab.json", "--vocab-size", "400", "--threads", "1"],
                   cwd=OUT, check=True, stdout=subprocess.DEVNULL)
    run_driver(["--save", "start.bin"], OUT)
    scratch = os.path.join(OUT, "_scratch.bin")
    _, eval_loss = run_driver(["--resume", "start.bin", "--save", scratch, "--test-file", "corpus.txt", "--lr", "0"], OUT)
    train = [run_driver(["--resume", "start.bin", "--save", scratch, "--lr", "0.001"], OUT)[0] for _ in range(3)]
    os.remove(scratch)
    with open(os.path.join(OUT, "expected.json"), "w") as f:
        json.dump({"model_args": MODEL_ARGS, "eval_loss": eval_loss, "train_loss": train}, f, indent=1)
    print("eval_loss", eval_loss, "train_loss", train)


if __name__ == "__main__":
    sys.exit(main())
