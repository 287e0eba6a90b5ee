"""Import the unmodified reference implementation (a copy under ``baseline/_ref``) as a CPU
oracle: all of its CUDA switches are turned off so its pure-PyTorch fallbacks define the
expected numbers."""
import importlib
import os
import sys

import pytest

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def load_reference():
    if not os.path.isfile(os.path.join(REF_DIR, "loomformer.py")):
        pytest.skip("reference copy not present under baseline/_ref")
    sys.dont_write_bytecode = True
    if REF_DIR not in sys.path:
        sys.path.append(REF_DIR)
    # the reference's entry module shares its name with ours at the repo root: import by path
    spec = importlib.util.spec_from_file_location("ref_loomformer", os.path.join(REF_DIR, "loomformer.py"))
    if "ref_loomformer" in sys.modules:
        return sys.modules["ref_loomformer"]
    tria_spec = importlib.util.spec_from_file_location("tria", os.path.join(REF_DIR, "tria.py"))
    tria_mod = importlib.util.module_from_spec(tria_spec)
    sys.modules["tria"] = tria_mod
    tria_spec.loader.exec_module(tria_mod)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_loomformer"] = mod
    spec.loader.exec_module(mod)
    return mod


def ref_config(lf, **kw):
    base = dict(use_cuda_phase_sin=False, use_cuda_beta_space=False, use_cuda_pvpowlu=False,
                use_cuda_depth_attn=False, use_cuda_tria=False, amp_dtype="fp32", attn_impl="manual")
    base.update(kw)
    return lf.Config(**base)
