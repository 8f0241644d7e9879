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


if __name__ == "__main__":
    main()
