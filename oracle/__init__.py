"""CPU restatement of the reference's operator set -- TEST INFRASTRUCTURE ONLY.

This package restates, in plain torch-CPU/numpy, what the Helion kernel bodies of
the reference (``helion_mlir_utils/*.py`` of adam-smnk/helion-mlir-xsmm) compute,
so that the CUDA kernels can be checked against it. It is imported only by
``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline legs.
The product (``helion_mlir_backend`` / ``helion_mlir_utils`` / ``libb200ops.so``)
never imports it and has no CPU path.

How it is pinned: the reference itself cannot be imported here (it needs
``helion``, MLIR bindings and ``lighthouse``, none installed), and its tests hold
no numeric golden vectors (they compare with eager torch). Two anchors are used:

* the layout formulas and tolerances of the reference's own tests
  (``tests/test_mlir_execution.py:1963-1981`` and the files cited per function);
* ``tests/golden/*.npz``: outputs of the reference's *own kernel bodies and host
  dispatch code* (``helion_mlir_utils``), executed eagerly under a small Helion
  stand-in by ``tests/golden/make_golden.py`` in the build container, where the
  reference source is mounted. ``tests/test_oracle.py`` checks this package
  against every fixture.

``rms_norm`` has no body and no test in the reference: its parity is unpinned
(the restatement follows torch's definition).
"""

from . import checks as checks
from . import inputs as inputs
from . import ops as ops
