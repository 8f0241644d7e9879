import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# data files of the fixture programs are found by name in this directory wherever the repository sits
# (the reference's compiled path honours the same variable: anvil/backend/anvil_host.h:134-141)
os.environ.setdefault("ANVIL_DATA", os.path.join(ROOT, "tests", "programs", "data"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
