"""Makes tests/golden/reference_model_logits.json with the reference's own model code.

prabanta-dev/janas runs quantized models only, so the whole model cannot be
compared on float weights.  But a tiny random Qwen3 whose matrices are exactly
what its eight-bit weight type holds (tests/golden/tiny_q8_model.py) can go
through its own tools on a CPU:

    the model as a GGUF file  ->  gguf2jns  ->  llm_eval ... dump=   (tests/llm_eval.c:7-20)

and the logits it writes are what its forward pass (src/llm/model.c:587) makes of
those weights.  They are not the float32 model's exactly: the reference rounds
the activations in front of every matrix product and the keys and values in its
cache to eight bits (src/llm/model_attn.c:42-48,115-145), which moves a logit by
about a hundredth of the largest.  tests/test_plain.py compares the plain
implementation with them within that; a wrong order of the parts, a wrong
pairing of heads, a norm in the wrong place would move them by as much as the
logits themselves.

    python tests/golden/make_model_golden.py /path/to/prabanta-dev/janas [--built DIR]

The reference is copied to a scratch folder and built there with its own
``./build.sh release`` (gcc; about ten minutes); ``--built DIR`` names a folder
that already holds ``gguf2jns`` and ``llm_eval`` instead.  Positions 0, 1, 7, 15,
23, 31, 38 and 39 of a 40-token sequence are kept, all 320 logits of each.
"""
import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import tiny_q8_model as tiny  # noqa: E402

KEEP = [0, 1, 7, 15, 23, 31, 38, 39]


def _string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str) -> None:
    """GGUF version 3 (src/llm/gguf.c:6-9): header, key-value pairs, tensor table,
    data from the next multiple of 32.  Value types: 4 uint32, 6 float32, 8 string;
    tensor types: 0 float32, 8 Q8_0."""
    c = tiny.CONFIG
    u32 = lambda k, v: _string(k) + struct.pack("<II", 4, v)
    f32 = lambda k, v: _string(k) + struct.pack("<If", 6, v)
    text = lambda k, v: _string(k) + struct.pack("<I", 8) + _string(v)
    kvs = [text("general.architecture", "qwen3"), text("general.name", "tiny random qwen3"),
           u32("general.alignment", 32), u32("qwen3.block_count", c["num_hidden_layers"]),
           u32("qwen3.context_length", c["max_position_embeddings"]),
           u32("qwen3.embedding_length", c["hidden_size"]),
           u32("qwen3.feed_forward_length", c["intermediate_size"]),
           u32("qwen3.attention.head_count", c["num_attention_heads"]),
           u32("qwen3.attention.head_count_kv", c["num_key_value_heads"]),
           u32("qwen3.attention.key_length", c["head_dim"]),
           u32("qwen3.attention.value_length", c["head_dim"]),
           f32("qwen3.attention.layer_norm_rms_epsilon", c["rms_norm_eps"]),
           f32("qwen3.rope.freq_base", c["rope_theta"])]
    tensors = tiny.tensors()
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)) + b"".join(kvs)
    infos, data = b"", bytearray()
    for name, _, w, raw, quantized in tensors:
        data += b"\0" * ((len(data) + 31) // 32 * 32 - len(data))
        dims = list(reversed(w.shape))               # the row's length first
        infos += _string(name) + struct.pack("<I", len(dims))
        infos += b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", 8 if quantized else 0, len(data))
        data += raw
    blob = head + infos
    blob += b"\0" * ((len(blob) + 31) // 32 * 32 - len(blob))
    with open(path, "wb") as f:
        f.write(blob + bytes(data))


def main() -> None:
    args = sys.argv[1:]
    built = None
    if "--built" in args:
        i = args.index("--built")
        built = args[i + 1]
        del args[i:i + 2]
    if len(args) != 1:
        sys.exit(__doc__)
    ref = args[0]
    here = os.path.dirname(os.path.abspath(__file__))
    with tempfile.TemporaryDirectory() as tmp:
        env = dict(os.environ, HOME=tmp)      # the reference writes tuning notes below HOME
        if built is None:
            src = os.path.join(tmp, "janas")
            shutil.copytree(ref, src)
            subprocess.run(["chmod", "-R", "u+w", src], check=True)
            print("building the reference (about ten minutes) ...", flush=True)
            subprocess.run(["./build.sh", "release"], cwd=src, check=True, env=env,
                           stdout=subprocess.DEVNULL)
            bins = os.path.join(src, "bin")
            built = os.path.join(bins, sorted(os.listdir(bins))[0])
        gguf, jns = os.path.join(tmp, "tiny.gguf"), os.path.join(tmp, "tiny.jns")
        toks, dump = os.path.join(tmp, "tokens.int32"), os.path.join(tmp, "logits.f32")
        write_gguf(gguf)
        np.asarray(tiny.TOKENS, dtype="<i4").tofile(toks)
        subprocess.run([os.path.join(built, "gguf2jns"), gguf, jns], check=True, env=env,
                       stdout=subprocess.DEVNULL)
        # no reference logits (-), 64 MiB of cache, two compute and two reader threads
        subprocess.run([os.path.join(built, "llm_eval"), jns, toks, "-", "64", "0,1", "2,3",
                        "dump=" + dump], check=True, env=env, stdout=subprocess.DEVNULL)
        logits = np.fromfile(dump, dtype="<f4").reshape(len(tiny.TOKENS), tiny.CONFIG["vocab_size"])
    out = {"positions": KEEP,
           "logits": [[round(float(v), 6) for v in logits[p]] for p in KEEP]}
    path = os.path.join(here, "reference_model_logits.json")
    with open(path, "w") as f:
        json.dump(out, f)
        f.write("\n")
    print("wrote", path, "largest logit", float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
