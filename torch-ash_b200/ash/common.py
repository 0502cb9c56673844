"""Loader of the native module and small utilities (API of ash/common.py)."""
import importlib


def _get_c_extension():
    """Return the native module ``__ash`` (the sm_100a C-ABI shim).

    The reference warns and carries on with ``None`` when its extension is
    missing (ash/common.py:4-16).  Here a missing library is an error: there is
    no CPU or eager fallback to carry on with.
    """
    try:
        mod = importlib.import_module("__ash")
    except ImportError as e:
        raise ImportError(
            "the native module `__ash` (libashb200.so) could not be loaded; "
            "build it with `python torch-ash_b200/build.py`"
        ) from e
    if not hasattr(mod, "HashMap"):
        raise ImportError(f"`__ash` at {getattr(mod, '__file__', '?')} is not the torch-ash native module")
    return mod


class DotDict(dict):
    """dict with attribute access (ash/common.py:19-22)."""

    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __setattr__(self, name, value):
        self[name] = value

    def __delattr__(self, name):
        try:
            del self[name]
        except KeyError:
            raise AttributeError(name) from None
