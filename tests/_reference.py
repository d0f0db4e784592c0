"""Loads the UNMODIFIED reference extensions from baseline/_ref (built by baseline/install_ref.sh) without
disturbing this repository's packages of the same names.  Test / bench infrastructure only."""
import importlib
import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
_cache = {}


def available():
    return os.path.isdir(os.path.join(REF_DIR, "dconv_native"))


def load(name):
    """name: 'dconv_native' or 'fast_depthwise_conv3d' -> the reference package (or None)."""
    if name in _cache:
        return _cache[name]
    if not available():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    saved = {k: v for k, v in sys.modules.items() if k == name or k.startswith(name + ".")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, REF_DIR)
    try:
        mod = importlib.import_module(name)
        assert os.path.abspath(mod.__file__).startswith(REF_DIR), mod.__file__
    except Exception:
        mod = None
    finally:
        sys.path.remove(REF_DIR)
        for k in [k for k in sys.modules if k == name or k.startswith(name + ".")]:
            del sys.modules[k]
        sys.modules.update(saved)
    _cache[name] = mod
    return mod
