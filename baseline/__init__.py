"""Access to the unmodified reference package installed by baseline/install_ref.py (comparison runs only)."""
from __future__ import annotations

import importlib
import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "hbsattn", "hbsa_interface.py"))


def load_reference():
    """Imports the reference's `hbsattn` package from baseline/_ref and returns the module.  Raises
    ImportError when it is not installed, or when the name `hbsattn` is already taken in this process by
    something else (hbsattn_b200.install_as_hbsattn registers the B200 package under that name)."""
    if not reference_available():
        raise ImportError("baseline/_ref is not installed (run baseline/install_ref.py with HBSATTN_REFERENCE set)")
    mod = sys.modules.get("hbsattn")
    if mod is not None:
        path = os.path.abspath(getattr(mod, "__file__", "") or "")
        if not path.startswith(REF_DIR):
            raise ImportError("the module name hbsattn is already bound to %s in this process" % path)
        return mod
    sys.path.insert(0, REF_DIR)
    try:
        return importlib.import_module("hbsattn")
    finally:
        sys.path.remove(REF_DIR)
