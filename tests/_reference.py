"""Locates an importable copy of the reference package (NovaNN) for the drop-in tests.

A pip-installed copy under ``baseline/_ref`` (git-ignored, made with ``pip install --target
baseline/_ref``) travels with the working tree; ``NOVANN_REFERENCE`` may name another directory
that holds the ``novann`` package.  Whichever is present is put on ``sys.path``; tests skip when
neither is.
"""
import logging
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CANDIDATES = [os.path.join(ROOT, "baseline", "_ref"), os.environ.get("NOVANN_REFERENCE", "")]


def import_novann():
    """Returns the imported ``novann`` package or None."""
    if "novann" in sys.modules:
        return sys.modules["novann"]
    for c in CANDIDATES:
        if c and os.path.isdir(os.path.join(c, "novann")):
            sys.path.insert(0, c)
            os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
            sys.dont_write_bytecode = True
            try:
                import novann
                logging.getLogger().setLevel(logging.WARNING)
                for name in list(logging.root.manager.loggerDict):
                    if "novann" in name.lower():
                        logging.getLogger(name).setLevel(logging.WARNING)
                return novann
            except Exception:
                sys.path.remove(c)
    return None
