"""Regenerates tests/golden/workload_<name>.npz from the reference itself.

Run where the reference checkout is present (it is compiled in place into oracle/_ref by
oracle/Makefile):  python tests/golden/make_golden.py

For every row of the five workloads it stores what the reference's own Generate() decided
(token id, log-prob, status), what the plain-C restatement reports beside it (survivor count,
distance of the draw from its CDF bucket edges, distance of the top-p walk from its cut), and a
checksum of the generated logits so a drifting generator is noticed.  Inputs are not stored: the
seeded generator rebuilds them.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path[:0] = [str(HERE.parent.parent), str(HERE.parent)]

import oracle_lib  # noqa: E402
import workload_rows  # noqa: E402
from pulsatrix_b200.workloads import WORKLOADS  # noqa: E402


def main():
    for name, w in WORKLOADS.items():
        out = {k: [] for k in ("token", "log_prob", "status", "survivors", "draw_margin", "top_p_margin", "u",
                               "checksum")}
        cfg = workload_rows.config_of(w)
        for start in range(0, w.rows, 64):
            ids = np.arange(start, min(start + 64, w.rows))
            logits, hist, offsets, seeds = workload_rows.build(name, ids)
            ref = oracle_lib.rows("reference", logits, hist, offsets, cfg, seeds, threads=8)
            orc = oracle_lib.rows("oracle", logits, hist, offsets, cfg, seeds, threads=8)
            assert (ref["token"] == orc["token"]).all(), f"{name}: restatement and reference disagree on a token"
            assert (ref["log_prob"] == orc["log_prob"]).all(), f"{name}: log-probs differ"
            assert (ref["status"] == 0).all()
            out["token"].append(ref["token"])
            out["log_prob"].append(ref["log_prob"])
            out["status"].append(ref["status"])
            for k in ("survivors", "draw_margin", "top_p_margin", "u"):
                out[k].append(orc[k])
            out["checksum"].append(np.array([workload_rows.logits_checksum(row) for row in logits], dtype=np.uint64))
        arrays = {k: np.concatenate(v) for k, v in out.items()}
        np.savez_compressed(HERE / f"workload_{name}.npz", **arrays)
        print(name, "rows", w.rows, "min draw margin", arrays["draw_margin"].min(), "min top-p margin",
              arrays["top_p_margin"].min(), "max survivors", arrays["survivors"].max())


if __name__ == "__main__":
    main()
