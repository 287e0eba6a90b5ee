#!/usr/bin/env python3
"""Command-line front end of ``loomformer_paraplex_b200.utils.slots`` (same flags as the reference's ``utils/analyze_tria_slots_pool.py``)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from loomformer_paraplex_b200.utils.slots import main  # noqa: E402

if __name__ == "__main__":
    main()
