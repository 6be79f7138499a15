"""Small stand-alone ETX programs that exercise the event protocol on the device (the reference keeps its own under
etx/operators/): the split-K row sum.  Each module follows the program protocol build() / bindings() / runtime()."""
from . import splitk_sum

__all__ = ["splitk_sum"]
