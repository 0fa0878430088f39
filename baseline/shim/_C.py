"""`qengine._C` served by this repository's library: every operator of the reference's BF16
extension (csrc/bindings.cpp of the reference) under the same name and argument order."""
import sys
from pathlib import Path

_REPO = Path(__file__).resolve().parents[5]
if str(_REPO) not in sys.path:
    sys.path.insert(0, str(_REPO))

from qengine_b200._C import *  # noqa: E402,F401,F403
from qengine_b200 import _C as _impl  # noqa: E402

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
