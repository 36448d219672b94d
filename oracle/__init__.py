"""CPU oracles for the WTConv forward path.

TEST INFRASTRUCTURE ONLY.  Nothing in this directory is part of the product:
the package ``wtconv_b200`` never imports it, and the CUDA path raises when its
extension is missing instead of falling back to anything here.  Allowed users
are the test-suite, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` (as the checker / the timed CPU arm).

Two independent restatements of the reference algorithm live here:

* ``oracle.wtconv_torch`` -- op-for-op restatement with ``torch.nn.functional``
  grouped convolutions (same operator sequence as the reference modules
  ``wtconv/wtconv2d.py:38-87`` and ``wtconv/wtconv1d.py:38-87``); runs in any
  dtype, so it also reproduces the reference's bf16/fp16 rounding behaviour.
* ``oracle.wtconv_np`` -- closed-form float64 numpy restatement (Haar
  butterflies + explicit depthwise stencils) used as the "truth" run.

Parity pin: both are checked against golden vectors produced by the reference
modules themselves (imported unchanged, with a table-only ``pywt`` stand-in),
see ``tests/golden/make_golden.py`` and ``tests/test_oracle_golden.py``.
"""
