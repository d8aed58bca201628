"""CPU oracle for the MetalDSP hot path (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import
this package.  The product (``metalaudio_b200``) never does: it fails loudly when
its CUDA library is missing instead of falling back to anything here.

Parity status
-------------
The reference (Swift + Apple Accelerate/Metal) cannot be compiled or imported on
Linux, and its arithmetic lives in the closed vDSP framework, so this package is a
restatement of the reference's algorithms in numpy/scipy:

* ``reference_path`` follows Sources/MetalDSP/FFT.swift, STFT.swift and
  Convolution.swift step by step in float32 (the "port"), and
* ``float64`` is the double-precision definition of the same operations.

Pinned: the 256-point forward / round-trip vectors that the reference's own
``scripts/generate_references.py`` (``generate_fft_references``, numpy seed 42)
emits are committed under ``tests/golden`` and both restatements are checked
against them, together with every analytic known-answer the reference's XCTest
suites assert (impulse, DC, bin-k sine, Parseval, conjugate symmetry, identity
kernel convolution ...).

parity unpinned: the reference holds no golden vectors and no tight assertions
for STFT -> iSTFT reconstruction accuracy or for partitioned-convolution accuracy
against true linear convolution; for those two the float64 definition here is the
only pin.
"""
