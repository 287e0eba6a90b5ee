#!/usr/bin/env python3
"""loomcloner: donor-transplant tool (``--scan DONOR_DIR`` writes a matching YAML, ``--clone CONFIG_YAML --donor DIR``
builds the checkpoint).  Flags as the reference tool (``loomcloner.py:441-477`` there)."""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser(description="loomcloner: donor-transplant tool for LoomFormer")
    ap.add_argument("--scan", type=str, default=None, metavar="DONOR_DIR")
    ap.add_argument("--clone", type=str, default=None, metavar="CONFIG_YAML")
    ap.add_argument("--donor", type=str, default=None, help="donor dir (required with --clone)")
    ap.add_argument("--mapping", type=str, default=None, help="mappings/*.json; auto-detected if omitted")
    ap.add_argument("--mappings-dir", type=str, default=os.path.join(ROOT, "mappings"))
    ap.add_argument("--out", type=str, required=True)
    ap.add_argument("--steps", type=int, default=8000)
    ap.add_argument("--lr", type=float, default=3e-5)
    ap.add_argument("--paraplex-gate-proj", action="store_true")
    ap.add_argument("--final-norm", action="store_true", help="transplant donor's model.norm.weight onto ln_final")
    ap.add_argument("--dataset", type=str, default="./datasets/REPLACE_ME")
    a = ap.parse_args()
    if bool(a.scan) == bool(a.clone):
        raise SystemExit("pass exactly one of --scan DONOR_DIR or --clone CONFIG_YAML")
    from loomformer_paraplex_b200.tools import cloner as cl
    if a.scan:
        donor = cl.donor_config(a.scan)
        mapping = cl.load_json(a.mapping or cl.detect_mapping(donor, a.mappings_dir))
        text = cl.scan_to_yaml(donor, mapping, a.scan, os.path.join(a.scan, "tokenizer.json"), a.dataset, a.steps, a.lr,
                               a.paraplex_gate_proj, a.final_norm)
        with open(a.out, "w", encoding="utf-8") as fh:
            fh.write(text)
        print(f"[loomcloner] wrote {a.out} (mapping={mapping.get('family')})")
        return
    if not a.donor:
        raise SystemExit("--clone requires --donor DONOR_DIR")
    cl.clone(a.clone, a.donor, a.mapping or cl.detect_mapping(cl.donor_config(a.donor), a.mappings_dir), a.out)


if __name__ == "__main__":
    main()
