"""Loads the unmodified reference modules (read-only) under private names for oracle tests."""
import importlib.util
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CANDIDATES = [ROOT / "baseline" / "_ref"] + ([Path(os.environ["GRUBOROS_REFERENCE"])] if os.environ.get("GRUBOROS_REFERENCE") else [])


def reference_root():
    for c in CANDIDATES:
        if (c / "mingru" / "minLM.py").exists():
            return c
    return None


def load_reference_mingru():
    """Returns (ref_minGRU_module, ref_minLM_module) or None when the reference tree is not present."""
    root = reference_root()
    if root is None:
        return None
    sys.dont_write_bytecode = True
    saved = {k: sys.modules.get(k) for k in ("mingru", "mingru.minGRU", "mingru.minLM")}
    try:
        for k in saved:
            sys.modules.pop(k, None)
        pkg_spec = importlib.util.spec_from_file_location("mingru", root / "mingru" / "__init__.py",
                                                          submodule_search_locations=[str(root / "mingru")])
        pkg = importlib.util.module_from_spec(pkg_spec)
        sys.modules["mingru"] = pkg
        g_spec = importlib.util.spec_from_file_location("mingru.minGRU", root / "mingru" / "minGRU.py")
        gmod = importlib.util.module_from_spec(g_spec)
        sys.modules["mingru.minGRU"] = gmod
        g_spec.loader.exec_module(gmod)
        l_spec = importlib.util.spec_from_file_location("mingru.minLM", root / "mingru" / "minLM.py")
        lmod = importlib.util.module_from_spec(l_spec)
        sys.modules["mingru.minLM"] = lmod
        l_spec.loader.exec_module(lmod)
        return gmod, lmod
    finally:
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v
