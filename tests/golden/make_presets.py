"""Writes tests/golden/reference_presets.csv: the (batch_size, num_tokens, varlen, cu_seqlens) rows of the reference's
own test presets, tests/settings/varlen.csv and tests/settings/product.csv of FlashQLA, in one table with a `source`
column.  The GPU parity test tests/test_presets_gpu.py runs every row.

    python tests/golden/make_presets.py /path/to/FlashQLA
"""
import csv
import os
import sys


def main(ref_root):
    out_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_presets.csv")
    rows = []
    for name in ("varlen.csv", "product.csv"):
        with open(os.path.join(ref_root, "tests", "settings", name)) as f:
            for r in csv.DictReader(f):
                rows.append(dict(source=name, batch_size=r["batch_size"], num_tokens=r["num_tokens"], varlen=r["varlen"],
                                 cu_seqlens=r.get("cu_seqlens") or ""))
    with open(out_path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=["source", "batch_size", "num_tokens", "varlen", "cu_seqlens"])
        w.writeheader()
        w.writerows(rows)
    print(f"{len(rows)} rows -> {out_path}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
