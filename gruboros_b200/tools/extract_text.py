"""Parquet -> training corpus: writes the ``text`` column of every parquet file found under the given paths as
one byte stream of UTF-8 documents separated by NUL bytes (the corpus format ``train.py --data`` memory-maps;
same output as the reference's extract_text.py:1-82).

    python -m gruboros_b200.tools.extract_text DIR_OR_FILE... [-o corpus.bin] [--min-length N]
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path


def find_parquet_files(paths):
    found = []
    for p in map(Path, paths):
        if p.is_file() and p.suffix.lower() == ".parquet":
            found.append(p)
        elif p.is_dir():
            found.extend(sorted(p.glob("**/*.parquet")))
    return found


def extract(file_path, out, min_length: int = 0, column: str = "text") -> int:
    """Stream one parquet file batch by batch; returns the number of documents written."""
    import pyarrow.parquet as pq
    n = 0
    pf = pq.ParquetFile(file_path)
    for batch in pf.iter_batches(columns=[column], batch_size=4096):
        for text in batch.column(0).to_pylist():
            if isinstance(text, str) and len(text) >= min_length:
                out.write(text.encode("utf-8") + b"\0")
                n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Extract text fields from parquet files, NUL-delimited")
    ap.add_argument("paths", nargs="+")
    ap.add_argument("--min-length", type=int, default=0)
    ap.add_argument("--output", "-o", type=str, default=None)
    a = ap.parse_args(argv)
    files = find_parquet_files(a.paths)
    if not files:
        print("No parquet files found in the specified paths.", file=sys.stderr)
        return 1
    out = open(a.output, "wb") if a.output else sys.stdout.buffer
    total = 0
    try:
        for i, f in enumerate(files, 1):
            try:
                n = extract(f, out, a.min_length)
            except Exception as exc:
                print(f"Error processing {f}: {exc}", file=sys.stderr)
                n = 0
            total += n
            print(f"[{i}/{len(files)}] {f}: {n} texts", file=sys.stderr)
    finally:
        if a.output:
            out.close()
    print(f"Total texts processed: {total}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
