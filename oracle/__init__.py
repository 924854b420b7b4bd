"""CPU oracle for the FlashLoop int4 KV-residual decode path.

TEST INFRASTRUCTURE ONLY.  This package restates, in plain numpy, the arithmetic
of the reference's CPU/Torch code for the decode hot path.  It exists so that the
CUDA kernels can be checked against an independent implementation.  Only
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl
reference`` legs of ``bench.py`` may import it; the product package
``flashloop_b200`` never does and fails loudly when its CUDA library is missing.

Parity pin: the reference ships no golden vectors for this path (its only test
file holds four repository checks).  The oracle is therefore pinned against
outputs of the reference's own Python code executed on CPU; the script that
produced them and the resulting vectors live in ``tests/golden/``.

Every function cites the reference file:line it follows (paths are relative to
the reference project's root).
"""

from . import bf16, packing, selection, cache, fakequant  # noqa: F401
