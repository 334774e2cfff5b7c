"""Loading of the committed golden fixtures (tests/golden/*.npz, made by make_golden.py)."""
import glob
import json
import os

import numpy as np

import refdump
from alphasparse_b200.matrices import CsrMatrix


def golden_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(refdump.GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(refdump.GOLDEN_DIR, name + ".npz"))
    m = CsrMatrix(int(z["shape"][0]), int(z["shape"][1]), z["indptr"], z["indices"], z["values"])
    man = refdump.Manifest(json.loads(bytes(z["manifest"]).decode()), np.ascontiguousarray(z["blob"]))
    spec = bytes(z["spec"]).decode()
    return m, z["x"], spec, man
