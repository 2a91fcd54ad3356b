"""The reference's model file (format v4, include/neuralnet.cpp/model_serialization.hpp:33-52, 389-503) read and
written from Python, so that the fused trainer can start from a checkpoint the reference wrote and hand one back.

    [magic u32 "NNNN"] [version u32 = 4] [precision u8: 0 = f32] [spec_len u64] [spec: KeyValueRecord]
    [parameter matrices in GPTModel::parameters order: rows u64, cols u64, rows*cols f32, row-major]
    [extra-state matrices (none for a GPT)] [tokenizer_len u64] [tokenizer JSON]

KeyValueRecord (keyvalue_record.hpp:60-180): field count u32, then per field key_len u32, key, type u8
(0 uint, 1 string, 2 uint array), value_len u32, value; all little-endian.

The reference file holds no optimizer state; `save_training_state` / `load_training_state` below keep the whole
state of a GptTrainer (parameters, Adam moments, Muon velocity, step counter) in a format of this repository.
"""
import struct
from typing import Dict, List, Sequence, Tuple

import numpy as np

MAGIC = 0x4E4E4E4E
VERSION = 4

# field order of spec_to_kv (model_serialization.hpp:196-216); a file written here is byte-identical to the reference's
SPEC_FIELDS = ("type", "layer_dims", "d_model", "num_heads", "d_ff", "num_layers", "patch_size", "vocab_size", "seq_len",
               "pos_encoding", "activation", "norm_type")
MODEL_TYPE_GPT = 3            # ModelType::GPT (model_spec.hpp:48-55)


def _parse_kv(buf: bytes) -> Dict[str, object]:
    out, off = {}, 0
    (count,) = struct.unpack_from("<I", buf, off); off += 4
    for _ in range(count):
        (klen,) = struct.unpack_from("<I", buf, off); off += 4
        key = buf[off:off + klen].decode(); off += klen
        typ = buf[off]; off += 1
        (vlen,) = struct.unpack_from("<I", buf, off); off += 4
        val = buf[off:off + vlen]; off += vlen
        if typ == 0:
            out[key] = struct.unpack("<Q", val)[0]
        elif typ == 1:
            out[key] = val.decode()
        elif typ == 2:
            out[key] = list(struct.unpack(f"<{vlen // 8}Q", val))
    return out


def _serialize_kv(fields: Sequence[Tuple[str, object]]) -> bytes:
    out = [struct.pack("<I", len(fields))]
    for key, val in fields:
        k = key.encode()
        out.append(struct.pack("<I", len(k)) + k)
        if isinstance(val, str):
            v = val.encode()
            out.append(b"\x01" + struct.pack("<I", len(v)) + v)
        elif isinstance(val, (list, tuple)):
            out.append(b"\x02" + struct.pack("<I", 8 * len(val)) + struct.pack(f"<{len(val)}Q", *val))
        else:
            out.append(b"\x00" + struct.pack("<I", 8) + struct.pack("<Q", int(val)))
    return b"".join(out)


def read_model_file(path: str):
    """Returns (spec dict, list of fp32 matrices in file order, tokenizer bytes).  A GPT has no extra-state
    matrices, so every matrix in the file is a parameter."""
    buf = open(path, "rb").read()
    magic, version, precision = struct.unpack_from("<IIB", buf, 0)
    if magic != MAGIC:
        raise ValueError(f"{path}: not a neuralnet.cpp model file")
    if version < 4:
        raise ValueError(f"{path}: format v{version} (offset-based headers) is not supported; v4 or later is")
    if precision != 0:
        raise ValueError(f"{path}: written with 64-bit scalars; this engine holds fp32 master weights")
    off = 9
    (spec_len,) = struct.unpack_from("<Q", buf, off); off += 8
    spec = _parse_kv(buf[off:off + spec_len]); off += spec_len
    return spec, buf, off


def split_matrices(buf: bytes, off: int, shapes: Sequence[Tuple[int, int]]):
    """Reads one matrix per expected shape (read_matrix checks the stored shape against the model's) and then the
    tokenizer block.  Returns (matrices, tokenizer bytes)."""
    mats = []
    for (r, c) in shapes:
        rows, cols = struct.unpack_from("<QQ", buf, off); off += 16
        if (rows, cols) != (r, c):
            raise ValueError(f"Matrix shape mismatch: expected ({r}, {c}), got ({rows}, {cols})")
        n = rows * cols
        mats.append(np.frombuffer(buf, np.float32, n, off).reshape(rows, cols).copy()); off += 4 * n
    (tlen,) = struct.unpack_from("<Q", buf, off); off += 8
    tok = buf[off:off + tlen]
    if len(tok) != tlen:
        raise ValueError("Unexpected end while reading tokenizer data")
    return mats, tok


def write_model_file(path: str, spec: Dict[str, object], matrices: Sequence[np.ndarray], tokenizer: bytes = b""):
    kv = _serialize_kv([(k, spec[k]) for k in SPEC_FIELDS])
    with open(path, "wb") as f:
        f.write(struct.pack("<IIB", MAGIC, VERSION, 0))
        f.write(struct.pack("<Q", len(kv)) + kv)
        for m in matrices:
            m = np.ascontiguousarray(m, np.float32)
            f.write(struct.pack("<QQ", m.shape[0], m.shape[1]))
            f.write(m.tobytes())
        f.write(struct.pack("<Q", len(tokenizer)) + tokenizer)


def spec_of_config(cfg) -> Dict[str, object]:
    """ModelSpec of a GPT (text_train.cpp fills it this way): enum encodings of model_spec.hpp:24-45 are the ones
    GptConfig already uses (positions 0 learned / 1 sinusoidal / 2 ALiBi; activation 0 GeLU / 1 SwiGLU; norm 0
    layer / 1 RMS)."""
    return {"type": MODEL_TYPE_GPT, "layer_dims": [], "d_model": cfg.d_model, "num_heads": cfg.heads, "d_ff": cfg.d_ff,
            "num_layers": cfg.layers, "patch_size": 0, "vocab_size": cfg.vocab, "seq_len": cfg.seq, "pos_encoding": cfg.pos,
            "activation": cfg.act, "norm_type": cfg.norm}


def check_spec_against_config(spec: Dict[str, object], cfg):
    want = spec_of_config(cfg)
    for k in ("d_model", "num_heads", "d_ff", "num_layers", "vocab_size", "pos_encoding", "activation", "norm_type"):
        if int(spec.get(k, want[k])) != int(want[k]):
            raise ValueError(f"checkpoint {k} = {spec.get(k)} does not match the trainer's {want[k]}")
    if cfg.pos == 0 and int(spec.get("seq_len", cfg.seq)) != cfg.seq:
        raise ValueError("learned position table length differs from the trainer's sequence length")


# ---------------------------------------------------------------- full training state (this repository's format)
STATE_MAGIC = b"NNB2STAT"


def save_training_state(path: str, arenas: Dict[str, np.ndarray], step: int, config_fields: Sequence[int]):
    """arenas: name -> flat fp32 array (params, adam_m, adam_v, muon_velocity as present)."""
    with open(path, "wb") as f:
        f.write(STATE_MAGIC + struct.pack("<QQ", step, len(config_fields)) + struct.pack(f"<{len(config_fields)}q", *config_fields))
        f.write(struct.pack("<Q", len(arenas)))
        for name, a in arenas.items():
            a = np.ascontiguousarray(a, np.float32).reshape(-1)
            nb = name.encode()
            f.write(struct.pack("<Q", len(nb)) + nb + struct.pack("<Q", a.size))
            f.write(a.tobytes())


def load_training_state(path: str):
    buf = open(path, "rb").read()
    if buf[:8] != STATE_MAGIC:
        raise ValueError(f"{path}: not a training-state file of this engine")
    step, ncfg = struct.unpack_from("<QQ", buf, 8)
    off = 24
    cfg = list(struct.unpack_from(f"<{ncfg}q", buf, off)); off += 8 * ncfg
    (count,) = struct.unpack_from("<Q", buf, off); off += 8
    arenas = {}
    for _ in range(count):
        (nl,) = struct.unpack_from("<Q", buf, off); off += 8
        name = buf[off:off + nl].decode(); off += nl
        (n,) = struct.unpack_from("<Q", buf, off); off += 8
        arenas[name] = np.frombuffer(buf, np.float32, n, off).copy(); off += 4 * n
    return arenas, int(step), cfg
