"""CPU oracle for the native Field recurrence. TEST INFRASTRUCTURE ONLY.

Two restatements of the reference's Field read live here:

* ``field_oracle.c`` (loaded through :mod:`oracle.field_oracle`): sequential
  double-precision recurrence, forward and backward, following
  ``field_only_v4_chunked_triton_wiki100.py:392-416`` and ``:794-909``.
* :mod:`oracle.torch_port`: the same arithmetic and the same scan shape as the
  reference's complex64 PyTorch path (``:333-416``), used as the timed CPU
  baseline.

Parity status: pinned against fixtures generated from the reference's own
``reference_field_read`` and autograd (``tests/golden/``).

Only tests, the smoke check and the benchmark's CPU-baseline / reference arm
may import this package. The shipped library never does.
"""
