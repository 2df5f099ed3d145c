"""Writes ``shipped_table_offsets.json``: the cumulative per-head counts (``kc_h_list``, ``kn_h_list``,
``vc_h_list``, ``vn_h_list``) of every ``_splithead`` dim table the reference ships under
``compressed_dims_file/`` -- the only part of those tables the decode planner looks at.  Needs a checkout of
the reference (first argument); the fixture it writes is what the tests read.

    python tests/golden/make_shipped_offsets.py <reference_dir>
"""
import glob
import json
import os
import sys


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = sys.argv[1]
    base = os.path.join(ref, "compressed_dims_file")
    out = {}
    for f in sorted(glob.glob(os.path.join(base, "*", "*_splithead.json"))):
        with open(f) as fh:
            d = json.load(fh)
        out[os.path.relpath(f, base)] = [{k: d[f"Layer_{i}"][k] for k in ("kc_h_list", "kn_h_list", "vc_h_list", "vn_h_list")}
                                         for i in range(len(d))]
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "shipped_table_offsets.json"), "w") as fh:
        json.dump(out, fh, separators=(",", ":"))
    print({k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
