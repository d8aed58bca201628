"""Regenerates the golden vectors committed in this folder from the reference's own
generator, ``scripts/generate_references.py`` (function ``generate_fft_references``,
``np.random.seed(42)`` set at import), equivalent to running that script with
``--operations fft``.  The reference tree does not travel to the GPU box, so the outputs
are committed: ``fft_forward_256.json`` and ``fft_roundtrip_256.json``.

With numpy >= 2 the generator's ``np.fft.fft`` of float32 input returns complex64, whose
float32 scalars the generator's plain ``json.dump`` cannot serialise; the generator's
``save_reference`` is therefore called through a ``json.dump`` that converts numpy scalars
with ``float()``.  The values are exactly what the generator computed.

Usage (where a checkout of the reference exists):
    python tests/golden/make_golden.py /path/to/reference
"""
import importlib.util
import json  # noqa: F401  (the generator's module-level json is patched below)
import os
import sys

here = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/reference")
ref_root = sys.argv[1]
path = os.path.join(ref_root, "scripts", "generate_references.py")
spec = importlib.util.spec_from_file_location("reference_generate_references", path)
mod = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mod)          # seeds numpy and torch with 42
_dump = mod.json.dump
mod.json.dump = lambda obj, f, **kw: _dump(obj, f, default=float, **kw)
mod.generate_fft_references(here)     # first draws after seeding, as with --operations fft
