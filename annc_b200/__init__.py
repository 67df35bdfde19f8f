"""annc_b200: B200 (sm_100a) implementation of the custom operators ANNC routes to.

The product is ``lib/libannc_b200.so`` (C ABI in ``include/annc_b200.h``); this Python
package is the thin host-side mirror used by the tests and the benchmark."""
from . import _lib  # noqa: F401  (fails loudly when the library is not built)
from ._lib import AnncError, lib  # noqa: F401

__all__ = ["AnncError", "lib"]
