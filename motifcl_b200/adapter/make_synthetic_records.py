"""Synthetic token records in the framing MotifCL's ternary15m trainer reads (tools/train_ternary15m.cpp:53-62,
124-131): DATA_DIR/train.bin and val.bin, little-endian uint16, records of seq+1 tokens.  The tokens are seeded
pseudo-random with a learnable rule (most transitions follow next = (31*cur + 7) mod 512), standing in for the
tokenised corpus the reference trained on, which is not part of either tree.

    python make_synthetic_records.py <dir> [seq=256] [train_records=4096] [val_records=128] [seed=1]
"""
import os
import sys

import numpy as np


def make_records(n_records: int, seq: int, seed: int, follow: float = 0.9, alphabet: int = 512) -> np.ndarray:
    rng = np.random.default_rng(seed)
    rec = np.empty((n_records, seq + 1), dtype=np.uint16)
    cur = rng.integers(0, alphabet, size=n_records)
    rec[:, 0] = cur
    for t in range(1, seq + 1):
        nxt = (31 * cur + 7) % alphabet
        jump = rng.random(n_records) >= follow
        nxt = np.where(jump, rng.integers(0, alphabet, size=n_records), nxt)
        rec[:, t] = nxt
        cur = nxt
    return rec


def write_dataset(out_dir: str, seq: int = 256, train_records: int = 4096, val_records: int = 128, seed: int = 1):
    os.makedirs(out_dir, exist_ok=True)
    make_records(train_records, seq, seed).astype("<u2").tofile(os.path.join(out_dir, "train.bin"))
    make_records(val_records, seq, seed + 1).astype("<u2").tofile(os.path.join(out_dir, "val.bin"))


if __name__ == "__main__":
    a = sys.argv[1:]
    write_dataset(a[0], *(int(v) for v in a[1:5]))
