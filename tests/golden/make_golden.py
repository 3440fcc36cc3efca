"""Generates tests/golden/*.npz from the REFERENCE's own code (oracle/_ref/libabq_ref.so, built from the reference's
engine/test_any_mma.cu by oracle/Makefile).  Run where the reference checkout is mounted:

    make -C oracle ref && python tests/golden/make_golden.py

Each fixture holds the inputs the reference generated with its own `init_matrix` (libc rand(), seed stated), the planes
packed by the CPU twin of its `pack` kernel, and the int32 output of its own `compute_ref`.  The fixtures are small on
purpose (a few KB each); they pin the oracle on machines where the reference is not mounted (the GPU box).
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

CASES = [
    # name, M, N, K, x_bits, w_bits, signed, seed
    ("w4a4_unsigned", 4, 48, 256, 4, 4, False, 1),
    ("w4a4_signed", 3, 40, 128, 4, 4, True, 1),
    ("w2a8_signed", 1, 96, 384, 8, 2, True, 7),
    ("w3a8_signed", 4, 32, 256, 8, 3, True, 11),
    ("w8a8_signed", 2, 24, 128, 8, 8, True, 3),
    ("w2a2_unsigned", 8, 16, 128, 2, 2, False, 5),
    ("w5a3_signed", 5, 33, 256, 3, 5, True, 9),
]


def main():
    assert O.ref_available(), "build oracle/_ref first (make -C oracle ref)"
    out = Path(__file__).resolve().parent
    for name, M, N, K, p, q, signed, seed in CASES:
        O.lib().abq_oracle_srand(seed)          # same libc generator state for the reference's init_matrix
        x = O.ref_init_matrix(M, K, p)          # the reference fills X first, then W (engine/test_any_mma.cu:127-128)
        w = O.ref_init_matrix(N, K, q)
        xp, wp = O.pack(x, p), O.pack(w, q)
        d = O.ref_compute_ref(wp, xp, signed)
        np.savez_compressed(out / f"{name}.npz", x=x.astype(np.int16), w=w.astype(np.int16), x_planes=xp, w_planes=wp, d=d,
                            meta=np.array([M, N, K, p, q, int(signed), seed], dtype=np.int32))
        print(name, d.shape, int(np.abs(d).max()))


if __name__ == "__main__":
    main()
