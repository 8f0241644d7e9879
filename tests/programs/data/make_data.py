"""Writes the small data files that tests/programs/data_files.anvil reads (seeded bytes in the IDX layout, a table
of numbers, a raw byte file). Synthetic: the shapes are those of a handwritten-digit set, the contents are random.

    python tests/programs/data/make_data.py
"""
import gzip
import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    rng = np.random.default_rng(2024)
    pix = rng.integers(0, 256, size=(6, 28, 28), dtype=np.uint8)
    lab = rng.integers(0, 10, size=(6,), dtype=np.uint8)
    with gzip.GzipFile(os.path.join(HERE, "images-idx3-ubyte.gz"), "wb", mtime=0) as f:       # magic: u8 elements, 3 dims
        f.write(struct.pack(">BBBBIII", 0, 0, 8, 3, 6, 28, 28) + pix.tobytes())
    with open(os.path.join(HERE, "labels-idx1-ubyte"), "wb") as f:
        f.write(struct.pack(">BBBBI", 0, 0, 8, 1, 6) + lab.tobytes())
    vals = rng.standard_normal((5, 4)).astype(np.float32)
    with open(os.path.join(HERE, "table.csv"), "w") as f:
        f.write("alpha,beta,gamma,delta\n")
        for row in vals:
            f.write(",".join("%.7g" % v for v in row) + "\n")
        f.write("-.5,+2e1,.25,7.\n")
    with open(os.path.join(HERE, "text.bin"), "wb") as f:
        f.write(rng.integers(0, 256, size=40, dtype=np.uint8).tobytes())


def write_corpus(path: str, nbytes: int = 24000, seed: int = 7):
    """A seeded pseudo-text (made-up words, sentence punctuation, line breaks) that stands in for the prose file a
    character-level language model trains on."""
    rng = np.random.default_rng(seed)
    letters = np.frombuffer(b"etaoinshrdlucmfwypvbgkq", dtype=np.uint8)
    words = ["".join(chr(c) for c in rng.choice(letters[:12 + rng.integers(0, 11)], size=rng.integers(2, 9))) for _ in range(300)]
    out, n, since = [], 0, 0
    while n < nbytes:
        w = words[int(rng.zipf(1.3)) % len(words)]
        since += 1
        if since > 6 and rng.random() < 0.2:
            w += rng.choice([".", ",", ";", "."])
            since = 0
        w += "\n" if rng.random() < 0.06 else " "
        out.append(w)
        n += len(w)
    with open(path, "wb") as f:
        f.write("".join(out).encode()[:nbytes])


def write_digit_set(directory: str, n: int = 60000, seed: int = 99):
    """`train-images-idx3-ubyte.gz` / `train-labels-idx1-ubyte.gz` with the layout and size of a handwritten-digit
    training set and seeded random contents (blurred blobs, so the pixel statistics are not white noise)."""
    rng = np.random.default_rng(seed)
    lab = rng.integers(0, 10, size=(n,), dtype=np.uint8)
    base = rng.integers(0, 256, size=(10, 28, 28)).astype(np.float32)
    for _ in range(2):                                              # smooth the ten class templates
        base = (base + np.roll(base, 1, 1) + np.roll(base, -1, 1) + np.roll(base, 1, 2) + np.roll(base, -1, 2)) / 5
    pix = np.clip(base[lab] + rng.integers(-40, 41, size=(n, 28, 28)), 0, 255).astype(np.uint8)
    with gzip.GzipFile(os.path.join(directory, "train-images-idx3-ubyte.gz"), "wb", compresslevel=1, mtime=0) as f:
        f.write(struct.pack(">BBBBIII", 0, 0, 8, 3, n, 28, 28) + pix.tobytes())
    with gzip.GzipFile(os.path.join(directory, "train-labels-idx1-ubyte.gz"), "wb", compresslevel=1, mtime=0) as f:
        f.write(struct.pack(">BBBBI", 0, 0, 8, 1, n) + lab.tobytes())


if __name__ == "__main__":
    main()
    write_corpus(os.path.join(HERE, "corpus.txt"))
