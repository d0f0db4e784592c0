"""Reads the per-unit timeline that an instrumented build of the forward kernel writes
(`python -m d2conv3d_b200.build --unit-trace`, then run any forward with D2C_UNIT_TRACE=<cta> set; see
csrc/deform_sm100_fwd_kernel.cuh for the buffer layout) and prints, per role, the mean clocks between its stamps,
and the distribution of the CTAs' durations.

    python -m d2conv3d_b200.unit_trace unit_trace_x3.bin
"""
import sys

import numpy as np

ROLES = ["record loader", "weight loader", "MMA issuer", "gather warp 0", "gather warp 15"]
STAMPS = [
    ["loop top", "stage free"],
    ["loop top", "stage free"],
    ["loop top", "A tile full", "weights full", "MMAs issued", "commits issued"],
    ["loop top", "row 1 loads issued", "A stage free", "row 0 blended", "next records there", "next row 0 loads issued",
     "row 1 blended", "arrived"],
]
STAMPS.append(STAMPS[3])


def main(path):
    raw = np.fromfile(path, dtype=np.int64)
    grid, k0 = int(raw[0]), int(raw[1])
    ev = raw[2:2 + 5 * 64 * 8].reshape(5, 64, 8)
    ctas = raw[2 + 5 * 64 * 8:2 + 5 * 64 * 8 + grid * 4].reshape(grid, 4)
    print(f"window: units {k0}..{k0 + 63} of the traced CTA (clock64 cycles)")
    for r, name in enumerate(ROLES):
        n = len(STAMPS[r])
        rows = ev[r][(ev[r][:, :n] > 0).all(axis=1)][:, :n]
        if len(rows) < 2:
            print(f"  {name}: no stamps")
            continue
        period = np.diff(rows[:, 0])
        print(f"  {name}: period per unit mean {period.mean():.0f} median {np.median(period):.0f}")
        seg = np.diff(rows, axis=1).mean(axis=0)
        for i in range(1, n):
            print(f"      {STAMPS[r][i - 1]:>24} -> {STAMPS[r][i]:<24} {seg[i - 1]:7.0f}")
    dur = (ctas[:, 1] - ctas[:, 0]) / 1e3
    t0 = ctas[:, 0].min()
    print(f"CTAs: {grid}, kernel span {(ctas[:, 1].max() - t0) / 1e3:.0f} us; CTA duration min {dur.min():.0f} "
          f"median {np.median(dur):.0f} mean {dur.mean():.0f} max {dur.max():.0f} us; units per CTA "
          f"{ctas[:, 3].min()}..{ctas[:, 3].max()}")
    for i in range(0, grid, 8):
        print("   cta %3d.. :" % i, " ".join("%5.0f" % d for d in dur[i:i + 8]))


if __name__ == "__main__":
    main(sys.argv[1])
