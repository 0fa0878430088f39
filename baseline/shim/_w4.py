"""`qengine._w4` served by this repository's library (the W4A16 GEMV of csrc/gemv_w4_bind.cpp of
the reference: gemv, gemv_swiglu, auto_ksplit with the same keywords)."""
import sys
from pathlib import Path

_REPO = Path(__file__).resolve().parents[5]
if str(_REPO) not in sys.path:
    sys.path.insert(0, str(_REPO))

from qengine_b200 import _w4 as _impl  # noqa: E402

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
