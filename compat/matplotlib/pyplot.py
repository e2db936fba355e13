"""No-op pyplot: ``imshow`` remembers the array and ``savefig`` writes it next to the requested
path as ``.npy`` (numeric error map instead of a picture)."""
import os

import numpy as np

_last = {"array": None}


def imshow(a, *args, **kwargs):
    _last["array"] = np.asarray(a)


def colorbar(*args, **kwargs):
    pass


def title(*args, **kwargs):
    pass


def scatter(*args, **kwargs):
    pass


def savefig(path, *args, **kwargs):
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    if _last["array"] is not None:
        np.save(os.path.splitext(path)[0] + ".npy", _last["array"])
