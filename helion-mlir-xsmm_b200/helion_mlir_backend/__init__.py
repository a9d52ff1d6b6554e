"""B200-native backend package with the reference's registration surface.

Importing it registers a Helion backend named ``"mlir"`` when Helion is
installed (:func:`install`), exactly as the reference's package does at import
(``helion_mlir_backend/__init__.py:38``); the operators of ``helion_mlir_utils``
run through :mod:`.native` either way.
"""

from __future__ import annotations

from . import output_pool as output_pool
from .api import compile_mlir as compile_mlir
from .api import generate_mlir as generate_mlir
from .api import lower_mlir as lower_mlir
from .call_trace import CallExplanation as CallExplanation
from .call_trace import explain as explain
from .driver import prepared_call as prepared_call
from .graphs import GraphedCall as GraphedCall
from .graphs import graphed as graphed
from .errors import MLIRBackendError as MLIRBackendError
from .errors import UnsupportedOperationError as UnsupportedOperationError
from .inject import install as install
from .language import InlineMLIRHint as InlineMLIRHint
from .language import inline_mlir as inline_mlir
from .native import set_native_call as set_native_call
from .output_pool import set_output_pool as set_output_pool

__all__ = [
    "CallExplanation",
    "GraphedCall",
    "InlineMLIRHint",
    "MLIRBackendError",
    "UnsupportedOperationError",
    "compile_mlir",
    "explain",
    "generate_mlir",
    "graphed",
    "inline_mlir",
    "install",
    "lower_mlir",
    "output_pool",
    "prepared_call",
    "set_native_call",
    "set_output_pool",
]

# Import-time side effect, as in the reference: make backend "mlir" available in Helion.
install()
