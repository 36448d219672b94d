"""Table-only stand-in for PyWavelets, for importing the reference in tests.

TEST INFRASTRUCTURE.  The reference reads only the four 2-tap db1 filter
vectors from ``pywt.Wavelet`` (wtconv/util/wavelet.py:7,24).  PyWavelets
(pinned 1.6.0 by the reference README) is not installable offline, so this
module tabulates those vectors; it implements no transform.  It is put on
``sys.path`` only by ``tests/golden/make_golden.py``.
"""
import math

_S = 1.0 / math.sqrt(2.0)
_TABLE = {
    "db1": dict(dec_lo=[_S, _S], dec_hi=[-_S, _S], rec_lo=[_S, _S], rec_hi=[_S, -_S]),
}
_TABLE["haar"] = _TABLE["db1"]


class Wavelet:
    def __init__(self, name):
        if name not in _TABLE:
            raise ValueError(f"pywt stand-in only tabulates db1/haar, got {name!r}")
        for k, v in _TABLE[name].items():
            setattr(self, k, list(v))
        self.name = name
