"""Turn the JSON a GPU test run leaves behind (``BG_PARITY_REPORT=<file> python -m pytest tests -m gpu``) into the
Markdown summary kept under ``profiles/``: per tolerance class the worst comparisons, and the comparisons closest to
their bound.

    python tests/parity_report_table.py <report.json> > profiles/parity_errors.md
"""
from __future__ import annotations

import json
import sys
from collections import defaultdict


def main(path: str) -> None:
    with open(path) as fh:
        rep = json.load(fh)
    rows = rep["comparisons"]
    floats = [r for r in rows if r["kind"] == "float"]
    exact = [r for r in rows if r["kind"] != "float"]
    print("# Parity errors measured by the GPU test run")
    print()
    print("Command: `BG_PARITY_REPORT=report.json python -m pytest tests -m gpu -q`, then "
          "`python tests/parity_report_table.py report.json`.")
    print(f"NumPy {rep['numpy']}; {len(rows)} comparisons against the oracle, the golden outputs of the unmodified reference or "
          f"another kernel of this build: {len(exact)} bit-exact, {len(floats)} under a tolerance.")
    print()
    print("Two errors per comparison: `max|d| / max|ref|` and the element-wise `max_i |d_i| / (|ref_i| + max|ref| * 2^-k)` "
          f"(k = {rep['floor_bits']['pointwise']} for pointwise graphs, {rep['floor_bits']['contraction']} for graphs with a "
          "contraction); both must stay below the case's rtol.")
    print()
    by_tol = defaultdict(list)
    for r in floats:
        by_tol[r["rtol"]].append(r)
    print("| rtol | comparisons | worst max-norm error | worst element-wise error | largest error / rtol |")
    print("|---|---|---|---|---|")
    for tol in sorted(by_tol):
        rs = by_tol[tol]
        worst = max(max(r["max_norm_err"], r["elementwise_err"]) for r in rs)
        print(f"| {tol:g} | {len(rs)} | {max(r['max_norm_err'] for r in rs):.2e} | {max(r['elementwise_err'] for r in rs):.2e} | "
              f"{worst / tol:.3f} |")
    print()
    print("Closest to their bound:")
    print()
    print("| comparison | dtype | elements | rtol | k | max-norm | element-wise | error / rtol |")
    print("|---|---|---|---|---|---|---|---|")
    key = lambda r: max(r["max_norm_err"], r["elementwise_err"]) / r["rtol"]
    seen = set()
    shown = 0
    for r in sorted(floats, key=key, reverse=True):
        if r["name"] in seen:
            continue
        seen.add(r["name"])
        print(f"| {r['name']} | {r['dtype']} | {r['numel']} | {r['rtol']:g} | {r['floor_bits']} | {r['max_norm_err']:.2e} | "
              f"{r['elementwise_err']:.2e} | {key(r):.3f} |")
        shown += 1
        if shown == 25:
            break


if __name__ == "__main__":
    main(sys.argv[1])
