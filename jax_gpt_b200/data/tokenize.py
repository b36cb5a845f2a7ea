"""Offline tokenizer: a directory of ``.txt`` files or a JSONL file with a ``text`` field ->
``train.bin`` / ``val.bin`` of uint16 GPT-2 BPE ids, one end-of-text token (50256) after every
document. As in the reference the validation split is the FIRST ``val_fraction`` of the token
stream (jax_gpt/data/tokenize_to_gcs.py:72-86).

    python -m jax_gpt_b200.data.tokenize --input corpus/ --output data/ --val_fraction 0.05

``--gcs_bucket/--gcs_path`` are accepted for command-line parity; uploading needs the
google-cloud-storage client, which is not part of this image.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

EOT_TOKEN = 50256


def iter_texts(input_path: str):
    if os.path.isfile(input_path):
        with open(input_path, "r", encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if line:
                    yield json.loads(line)["text"]
    elif os.path.isdir(input_path):
        for fname in sorted(os.listdir(input_path)):
            if fname.endswith(".txt"):
                with open(os.path.join(input_path, fname), "r", encoding="utf-8") as fh:
                    yield fh.read()
    else:
        raise FileNotFoundError(f"input path not found: {input_path}")


def get_encoder(name: str = "gpt2"):
    """tiktoken's GPT-2 BPE when its vocabulary is available offline, else a byte-level fallback
    (ids 0..255) so the pipeline stays usable without network access."""
    try:
        import tiktoken
        enc = tiktoken.get_encoding(name)
        enc.encode_ordinary("probe")
        return enc.encode_ordinary
    except Exception:
        return lambda text: list(text.encode("utf-8"))


def tokenize(input_path: str, val_fraction: float = 0.05, encode=None):
    encode = encode or get_encoder()
    ids = []
    for text in iter_texts(input_path):
        ids.extend(encode(text))
        ids.append(EOT_TOKEN)
    arr = np.asarray(ids, dtype=np.uint16)
    n_val = max(1, int(len(arr) * val_fraction))
    return arr[n_val:], arr[:n_val]


def write_split(arr: np.ndarray, output_dir: str, split: str) -> str:
    os.makedirs(output_dir, exist_ok=True)
    path = os.path.join(output_dir, f"{split}.bin")
    arr.tofile(path)
    print(f"Wrote {len(arr):,} tokens -> {path}")
    return path


def write_synthetic(output_dir: str, n_tokens: int, vocab_size: int = 50257, seed: int = 0, val_fraction: float = 0.05):
    """Uniform-random token ids, for benchmarks and smoke runs without a corpus."""
    rng = np.random.default_rng(seed)
    arr = rng.integers(0, vocab_size, size=n_tokens, dtype=np.uint16)
    n_val = max(1, int(n_tokens * val_fraction))
    return write_split(arr[n_val:], output_dir, "train"), write_split(arr[:n_val], output_dir, "val")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", default="")
    ap.add_argument("--gcs_bucket", default="")
    ap.add_argument("--gcs_path", default="")
    ap.add_argument("--val_fraction", type=float, default=0.05)
    ap.add_argument("--format", default="bin", choices=["bin"])
    args = ap.parse_args(argv)
    if not args.output and not args.gcs_bucket:
        ap.error("give --output and/or --gcs_bucket")
    train, val = tokenize(args.input, args.val_fraction)
    if args.output:
        write_split(train, args.output, "train")
        write_split(val, args.output, "val")
    if args.gcs_bucket:
        raise SystemExit("object-store upload needs google-cloud-storage, which is not installed; use --output")


if __name__ == "__main__":
    main()
