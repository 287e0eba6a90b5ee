#!/usr/bin/env python3
"""loompack: build, inspect and unpack ``.aio`` inference packages (sub-commands and flags as the reference tool,
``loompack.py:321-377`` there)."""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main(argv=None) -> int:
    from loomformer_paraplex_b200.serve import package as pk
    ap = argparse.ArgumentParser(prog="loompack.py")
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("pack")
    p.add_argument("model", help="LoomFormer .pt checkpoint")
    p.add_argument("--tokenizer", required=True, help="tokenizer JSON")
    p.add_argument("--template", required=True, help="chat template Jinja")
    p.add_argument("-o", "--output", required=True, help="output .aio")
    p.add_argument("--quant", default="none", help="none, fp32, bf16, or fp16")
    p.add_argument("--min-quant-elements", type=int, default=pk.DEFAULT_MIN_QUANT_ELEMENTS,
                   help=f"keep smaller tensors in fp32 (default: {pk.DEFAULT_MIN_QUANT_ELEMENTS})")
    p = sub.add_parser("inspect")
    p.add_argument("archive")
    p.add_argument("--keys", action="store_true")
    p = sub.add_parser("extract")
    p.add_argument("archive")
    p.add_argument("-d", "--directory", required=True)
    a = ap.parse_args(argv)
    if a.command == "pack":
        m = pk.build_package(a.model, a.tokenizer, a.template, a.output, a.quant, a.min_quant_elements)
        q = m["quantization"]
        print(f"[loompack] {a.output}: {m['model']['parameters']:,} params, quant={q['target_dtype']}, "
              f"tensors={q['changed_tensors']} converted, archive={pk.size_text(m['archive_bytes'])}")
        print(f"[loompack] tensor bytes: {pk.size_text(q['source_bytes'])} -> {pk.size_text(q['packed_tensor_bytes'])}")
    elif a.command == "inspect":
        pk.inspect_package(a.archive, show_keys=a.keys)
    else:
        pk.extract_package(a.archive, a.directory)
        print(f"[loompack] extracted to {a.directory}")
    return 0


if __name__ == "__main__":
    try:
        raise SystemExit(main())
    except (OSError, ValueError, TypeError, RuntimeError) as exc:
        print(f"loompack: {exc}", file=sys.stderr)
        raise SystemExit(1)
