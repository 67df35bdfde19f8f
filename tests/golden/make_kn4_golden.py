"""Generates tests/golden/kn4_golden.npz by running the reference's own packer.

Run in a container that has the reference tree:
    python tests/golden/make_kn4_golden.py <path of the ANNC checkout>
It loads python/annc/optimize/data_pack.py from that tree as a stand-alone module
(numpy only) and packs B = arange(K*N) with FormageChange(12).run(kn -> kn4,
tiles (0,352),(1,128)) exactly as python/annc/optimize/constant_folding.py:77-88
does.  Small shapes are stored whole (the packed buffer is then the permutation
itself); the large shapes are stored as a SHA-256 of the packed float32 bytes.
"""
import hashlib
import importlib.util
import os
import sys

import numpy as np

SMALL = [(12, 12), (13, 17), (30, 20), (352, 128), (353, 129), (400, 140), (705, 257),
         (64, 1), (1, 64), (24, 300)]
LARGE = [(2048, 4096), (1024, 1024), (416, 512), (1000, 1000)]


def main(ref_root: str) -> None:
    path = os.path.join(ref_root, "python/annc/optimize/data_pack.py")
    spec = importlib.util.spec_from_file_location("ref_data_pack", path)
    dp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dp)
    out = {}
    for K, N in SMALL + LARGE:
        B = np.arange(K * N, dtype=np.float32).reshape(K, N)
        packed = dp.FormageChange(12).run(
            B, dp.DataFormat.kn, dp.DataFormat.kn4,
            [dp.MatrixTiling(0, 352), dp.MatrixTiling(1, 128)])
        assert packed.shape == (K, N) and packed.dtype == np.float32
        if (K, N) in SMALL:
            out[f"perm_{K}x{N}"] = packed.reshape(-1).astype(np.int32)
        else:
            h = hashlib.sha256(np.ascontiguousarray(packed).tobytes()).hexdigest()
            out[f"sha_{K}x{N}"] = np.frombuffer(bytes.fromhex(h), dtype=np.uint8)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kn4_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ANNC_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_kn4_golden.py <ANNC checkout>  (or set ANNC_REFERENCE_ROOT)")
    main(root)
