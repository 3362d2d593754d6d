import os
import shutil
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle_mod():
    """The CPU checkers (restatement always; the compiled reference when it is present)."""
    import oracle
    subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)
    return oracle


@pytest.fixture(scope="session")
def native_lib():
    """The product library; built in-tree when nvcc is at hand and the sources are newer."""
    from openfish_b200 import build
    if shutil.which(build.NVCC) or os.path.exists(build.NVCC):
        build.build()
    import openfish_b200
    return openfish_b200


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    d = {k: z[k] for k in z.files}
    if "opt_keys" in d:
        d["options"] = {str(k): float(v) for k, v in zip(d.pop("opt_keys"), d.pop("opt_values"))}
        d["state_len"] = int(d["state_len"])
    return d


SYNTH_CASES = ["fast", "hac", "sup", "fast_c320", "fast_stays", "hac_cut10", "fast_temp07", "hac_temp16"]
# every array a fixture holds besides the scores (see tests/golden/make_golden.py)
FIXTURE_OUTPUTS = ("moves", "sequence", "qstring", "bwd", "fwdbwd", "post", "states", "qual", "base_probs",
                   "total_probs")
