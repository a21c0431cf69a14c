"""Generates tests/golden/fp8_e4m3_torch.npz: f32 bit patterns and the E4M3FN byte
torch.float8_e4m3fn assigns to each (the independent encoder the reference's
scripts/test_fp8_encode.py checks against).  Run once here; the .npz is committed.

    python tests/golden/make_fp8_vectors.py
"""
import os

import numpy as np
import torch


def main():
    g = np.random.default_rng(20240607)
    parts = [
        g.standard_normal(2048).astype(np.float32) * 100.0,          # bulk of the range
        g.standard_normal(1024).astype(np.float32),                  # around 1
        (g.standard_normal(1024) * 2.0 ** -8).astype(np.float32),    # subnormal zone
        g.uniform(-460, 460, 1024).astype(np.float32),               # saturation edge
    ]
    # every rounding tie between adjacent positive codes, and just either side of it
    codes = torch.arange(0, 0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    mids = (codes[:-1] + codes[1:]) / 2
    ties = np.concatenate([mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf))])
    parts += [ties.astype(np.float32), -ties.astype(np.float32), codes, -codes]
    x = np.concatenate(parts).astype(np.float32)
    x = x[np.isfinite(x)]
    enc = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    # torch maps |x| > 464 to NaN instead of saturating; keep only the range both agree on
    keep = np.abs(x) <= 448.0
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fp8_e4m3_torch.npz")
    np.savez_compressed(out, bits=x[keep].view(np.uint32), code=enc[keep], torch_version=torch.__version__)
    print(out, int(keep.sum()), "vectors")


if __name__ == "__main__":
    main()
