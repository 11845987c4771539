"""Generates the golden vectors in this directory from the reference's own host code.

Needs oracle/_ref/libttref.so, i.e. a container where the reference tree was present when
``oracle.build()`` ran. Usage:  python tests/golden/make_golden.py

Outputs
  bfp_golden.npz   packed bytes / unpacked fp32 bit patterns for the small known-answer inputs
  digests.json     SHA-256 of the reference's outputs on the larger seeded inputs
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402
import vectors  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    ref = oracle.ref()
    assert ref is not None, "oracle/_ref/libttref.so is missing: run oracle.build() where the reference tree exists"
    out, dig = {}, {}
    tile = vectors.arange_tile()
    adv = vectors.adversarial_bits()
    for fmt, name in ((0, "bfp8"), (1, "bfp4")):
        # the reference's own known-answer case: row-major-in pack must equal tilize-then-pack
        out[f"arange_{name}_packed"] = ref.pack(tile, fmt, in_tile_row_major=True)
        out[f"arange_{name}_unpacked_rm"] = ref.unpack(out[f"arange_{name}_packed"], fmt, in_tile_row_major=True).view(np.uint32)
        p = ref.pack(adv, fmt)
        out[f"adv_{name}_packed"] = p
        dig[f"adv_{name}_unpacked"] = sha(ref.unpack(p, fmt).view(np.uint32))
        dig[f"adv_{name}_from_torch_16x1024"] = sha(ref.from_torch(adv, fmt, 1, 16 * 32, 32))
        ex = vectors.exhaustive_packed(fmt)
        dig[f"exhaustive_{name}_unpacked"] = sha(ref.unpack(ex, fmt).view(np.uint32))
        dig[f"exhaustive_{name}_to_torch"] = sha(ref.to_torch(ex, fmt, 1, 256 * 32, 32).view(np.uint32))
        # seeded tensors of the benchmark configurations
        for label, seed, shape in (("c1_4096x4096_seed0", 0, (1, 4096, 4096)), ("rand_2x3x64x96_seed0", 0, (6, 64, 96)),
                                   ("c2_slice_256x512_seed1", 1, (1, 256, 512))):
            x = vectors.randn(seed, shape, 0.02).numpy()
            packed = ref.from_torch(x, fmt, *shape)
            dig[f"{label}_{name}_from_torch"] = sha(packed)
            dig[f"{label}_{name}_to_torch"] = sha(ref.to_torch(packed, fmt, *shape).view(np.uint32))
    t = np.arange(3 * 64 * 96, dtype=np.float32)
    dig["tilize_3x64x96_arange"] = sha(ref.tilize(t, 3, 64, 96))
    np.savez_compressed(os.path.join(HERE, "bfp_golden.npz"), **out)
    with open(os.path.join(HERE, "digests.json"), "w") as f:
        json.dump(dig, f, indent=1, sort_keys=True)
    print("wrote", len(out), "arrays and", len(dig), "digests")


if __name__ == "__main__":
    main()
