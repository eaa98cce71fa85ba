"""CPU oracle for the Hyena convolution path.

TEST INFRASTRUCTURE ONLY.  Nothing in ``vortex_b200`` imports this package.
It may be imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` -- there only as
the checker or as the timed CPU baseline, never as part of the product path.

Two restatements of the reference algorithm live here:

* ``hyena_oracle`` -- numpy, float64 accumulation, explicit rounding points.
  Independent arithmetic (direct sums, no FFT library on the FIR paths).
* ``torch_port``   -- the same operator sequence expressed with the library
  calls the reference itself uses on CPU (``F.conv1d`` / ``torch.fft``), used
  as the timed CPU baseline with all host threads.

Parity pin: both are checked against golden vectors produced by importing the
reference's own ``HyenaInferenceEngine`` (``vortex/model/engine.py``) -- see
``tests/golden/make_golden.py`` and ``tests/test_oracle_golden.py``.
"""
