"""The reader of the forward kernel's optional per-unit timeline (d2conv3d_b200/unit_trace.py) on a synthetic dump:
layout [grid, k0][5 roles x 64 units x 8 stamps][grid x {t0, t1, smid, units}] of int64, as the instrumented build
writes it (csrc/deform_sm100_fwd_kernel.cuh)."""
import numpy as np

from d2conv3d_b200 import unit_trace


def test_reader_reports_period_and_cta_durations(tmp_path, capsys):
    grid, k0 = 4, 200
    ev = np.zeros((5, 64, 8), dtype=np.int64)
    for role, stamps in enumerate((2, 2, 5, 8, 8)):
        for k in range(64):
            for e in range(stamps):
                ev[role, k, e] = 10_000 + 4_000 * k + 100 * e          # period 4000 clocks, 100 between stamps
    ctas = np.array([[1_000, 601_000, sm, 300] for sm in range(grid)], dtype=np.int64)    # 600 us each
    path = tmp_path / "trace.bin"
    np.concatenate([np.array([grid, k0], dtype=np.int64), ev.ravel(), ctas.ravel()]).tofile(path)
    unit_trace.main(str(path))
    out = capsys.readouterr().out
    assert "units 200..263" in out
    assert out.count("period per unit mean 4000 median 4000") == 5
    assert "CTA duration min 600 median 600 mean 600 max 600 us" in out
    assert "units per CTA 300..300" in out
